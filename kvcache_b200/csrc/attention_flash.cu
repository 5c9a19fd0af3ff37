// bfloat16 attention over cache pages on the tensor cores: a kernel for segments that bring
// few rows (decode: split over the keys, all query heads of a kv head in one warp) and a
// kernel for portions of prompts (64 query positions of one head per block).
//
// What they replace in the reference: k_batched_paged_decode_attn and k_paged_attn
// (src/qwen_kernels.cu:293-335, :146-185; one block of D threads per (query, head), serial
// over the keys with a tree reduction per key), with the split over the keys and its merge
// taken from the toy flash-decode kernel (src/flash_decode.cu:18-101).
#include "flash_core.cuh"
#if KVB_HEAD_DIM % 64 == 0
#include "tc_common.cuh"
#endif

using namespace flash;

#define DECODE_STAGES (KVB_HEAD_DIM <= 64 ? 3 : 2)
#define PREFILL_STAGES 2
#define PREFILL_MAX_UNITS 16

// ---------------------------------------------------------------------------------------------
// Decode: one block of four warps per (item, kv head, split).  An item is a segment whose
// rows * group <= 16: row r is query (r / G) of the segment, head hk * G + r % G, so keys and
// values are read once for all heads that share them.  The block scans a range of key tiles;
// of every 64-key tile each warp takes 16 keys and keeps its own running (m, l, acc), the four
// are merged through shared memory at the end.  With several splits the block leaves
// (m, l, acc) in scratch and the last block to finish (a ticket counter per (item, kv head))
// merges the splits in order and resets the counter.
// ---------------------------------------------------------------------------------------------
struct DecodeParams {
    const bf16* q;             // [T, Hq * D]
    bf16* out;                 // [T, Hq * D]
    const bf16* k_pages;
    const bf16* v_pages;
    const int* block_table;    // [segments, table_stride]
    const int* items;          // segment of each item, or nullptr: item i is segment i
    const int* seg_q_start;
    const int* seg_q_len;
    const int* seg_kv_len;
    float* part_o;             // [items, Hkv, nsplit, 16, D]
    float* part_ml;            // [items, Hkv, nsplit, 16, 2]
    int* tickets;              // [items, Hkv], zero between launches
    int table_stride, Hq, Hkv, page_size, page_shift, window, nsplit;
    float scale_log2;
    int nsuper;                // TMA kernel: clusters per (item, kv head), each with its own run of keys (1: the cluster is all)
};

constexpr int MAX_SPLITS = 32;


__global__ void __launch_bounds__(128) flash_decode_kernel(const DecodeParams p) {
    TRACE(0)
    pdl_wait();
    pdl_launch_dependents();
    TRACE(1)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int ticket_s;
    const int split = blockIdx.x, hk = blockIdx.y, item = blockIdx.z;
    const int seg = p.items ? p.items[item] : item;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = p.Hq / p.Hkv;
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int rows = min(q_len * G, 16);   // an item is one warp tile of 16 rows; rows beyond it are not this kernel's (see no_alloc.h)
    const int first_pos = kv_len - q_len;
    const int key_lo = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
    const int tile_begin = key_lo / KT, tile_end = (kv_len + KT - 1) / KT;
    const int num_tiles = tile_end - tile_begin;
    const int per_split = (num_tiles + p.nsplit - 1) / p.nsplit;
    const int n_valid = (num_tiles + per_split - 1) / per_split;       // splits that have tiles
    if (split >= n_valid) return;
    const int my_begin = tile_begin + split * per_split;
    const int my_end = min(tile_end, my_begin + per_split);
    const int n = my_end - my_begin;

    KVSource src{p.k_pages, p.v_pages, p.block_table + (size_t)seg * p.table_stride, hk, p.Hkv, p.page_size, p.page_shift};
    WarpRows w;
    rows_init(w);
    auto q_row = [&](int r) -> const bf16* {
        return r < rows ? p.q + ((size_t)(q_start + r / G) * p.Hq + hk * G + r % G) * D : nullptr;
    };
    rows_load_q(w, q_row);
    w.pos[0] = g < rows ? first_pos + g / G : -1;
    w.pos[1] = g + 8 < rows ? first_pos + (g + 8) / G : -1;

    constexpr int STAGES = DECODE_STAGES;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n) load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (my_begin + s) * KT, key_lo, kv_len);
        cp_async_commit();
    }
    for (int i = 0; i < n; ++i) {
        const int ahead = i + STAGES - 1;
        if (ahead < n) {
            const int s = ahead % STAGES;
            load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (my_begin + ahead) * KT, key_lo, kv_len);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (i == 0) { TRACE(2) }
        const int s = i % STAGES;
        // Of every tile each warp takes 16 keys and keeps its own running (m, l, acc).  Rows that do not
        // exist (beyond rows) have zero queries and are never stored, so only the positions of existing rows
        // decide whether the keys need their mask.
        {
            const int key0 = (my_begin + i) * KT + warp * 16;
            if (key0 < kv_len)
                rows_tile_auto<16>(w, smem + (2 * s) * TILE_ELEMS + warp * 16 * STRIDE,
                                   smem + (2 * s + 1) * TILE_ELEMS + warp * 16 * STRIDE, key0, p.window, p.scale_log2,
                                   first_pos, kv_len - 1, true);
        }
        __syncthreads();
    }
    rows_finish_sum(w);
    TRACE(3)

    // The four warps' results meet in shared memory (the stages are free now).
    float* wo = reinterpret_cast<float*>(smem_raw);            // [4][16][D]
    float* wml = wo + 4 * 16 * D;                              // [4][16][2]
    float* wgt = wml + 4 * 16 * 2;                             // [16][MAX_SPLITS] weights of the split merge
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int i = 0; i < NT_O; ++i)
            *reinterpret_cast<float2*>(wo + (warp * 16 + row) * D + i * 8 + 2 * t) = make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
        if (t == 0) { wml[(warp * 16 + row) * 2] = w.m[r]; wml[(warp * 16 + row) * 2 + 1] = w.l[r]; }
    }
    __syncthreads();
    const size_t slot = ((size_t)item * p.Hkv + hk) * p.nsplit;
    for (int idx = tid; idx < rows * D; idx += 128) {
        const int row = idx / D, d = idx - row * D;
        float M = NEG_INF;
#pragma unroll
        for (int x = 0; x < 4; ++x) M = fmaxf(M, wml[(x * 16 + row) * 2]);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const float e = exp2f(wml[(x * 16 + row) * 2] - base);
            L += e * wml[(x * 16 + row) * 2 + 1];
            acc += e * wo[(x * 16 + row) * D + d];
        }
        if (n_valid == 1) {
            p.out[((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            p.part_o[((slot + split) * 16 + row) * D + d] = acc;
            if (d == 0) {
                p.part_ml[((slot + split) * 16 + row) * 2] = M;
                p.part_ml[((slot + split) * 16 + row) * 2 + 1] = L;
            }
        }
    }
    if (n_valid == 1) return;

    // Take a ticket; the last block of this (item, kv head) merges the splits.
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket_s = atomicAdd(p.tickets + item * p.Hkv + hk, 1);
    __syncthreads();
    TRACE(4)
    if (ticket_s != n_valid - 1) return;
    __threadfence();
    if (tid == 0) p.tickets[item * p.Hkv + hk] = 0;
    // weight[row][s] = 2^(m_s - M) / sum_s 2^(m_s - M) l_s; out[row][d] = sum_s weight[row][s] acc_s[row][d],
    // added in split order.  Loads are issued many at a time: this block is alone with their latency.
    float* mls = wgt + 16 * MAX_SPLITS;                        // [16][MAX_SPLITS][2]
    for (int idx = tid; idx < rows * n_valid; idx += 128) {
        const int row = idx / n_valid, s = idx - row * n_valid;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((slot + s) * 16 + row) * 2));
        mls[(row * MAX_SPLITS + s) * 2] = ml.x;
        mls[(row * MAX_SPLITS + s) * 2 + 1] = ml.y;
    }
    __syncthreads();
    if (tid < rows) {
        const int row = tid;
        float M = NEG_INF;
        for (int s = 0; s < n_valid; ++s) M = fmaxf(M, mls[(row * MAX_SPLITS + s) * 2]);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f;
        for (int s = 0; s < n_valid; ++s) {
            const float e = exp2f(mls[(row * MAX_SPLITS + s) * 2] - base);
            L += e * mls[(row * MAX_SPLITS + s) * 2 + 1];
            wgt[row * MAX_SPLITS + s] = e;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int s = 0; s < n_valid; ++s) wgt[row * MAX_SPLITS + s] *= inv;
    }
    __syncthreads();
    TRACE(5)
    for (int idx = tid; idx < rows * (D / 4); idx += 128) {
        const int row = idx / (D / 4), d = (idx - row * (D / 4)) * 4;
        const float* po = p.part_o + (slot * 16 + row) * D + d;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < n_valid; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int x = 0; x < 8; ++x)
                v[x] = s0 + x < n_valid ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)(s0 + x) * 16 * D))
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const float ws = s0 + x < n_valid ? wgt[row * MAX_SPLITS + s0 + x] : 0.f;
                acc.x += ws * v[x].x; acc.y += ws * v[x].y; acc.z += ws * v[x].z; acc.w += ws * v[x].w;
            }
        }
        bf16* o = p.out + ((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d;
        *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
    TRACE(6)
}

// Bytes of scratch for `items` items: partial outputs, partial (m, l), tickets.
KVB_API int kvb_flash_head_dim() { return D; }

KVB_API long long kvb_flash_decode_scratch_floats(int items, int Hkv, int nsplit) {
    return (long long)items * Hkv * nsplit * 16 * (D + 2);
}

// `scratch`: kvb_flash_decode_scratch_floats floats; `tickets`: items * Hkv ints, zero before the
// first launch (the kernel leaves them zero).
KVB_API int kvb_flash_decode(const void* q, void* out, const void* k_pages, const void* v_pages,
                             const int* block_table, int table_stride, const int* items, int n_items,
                             const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, float* scratch,
                             int* tickets, int Hq, int Hkv, int page_size, int window, int nsplit, float scale,
                             cudaStream_t stream) {
    if (n_items <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (nsplit < 1 || nsplit > MAX_SPLITS || n_items > 65535 || Hkv > 65535) return KVB_ERR_LIMIT;
    DecodeParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.items = items; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)n_items * Hkv * nsplit * 16 * D;
    p.tickets = tickets;
    p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.nsplit = nsplit;
    p.scale_log2 = scale * 1.4426950408889634f;
    size_t smem = (size_t)DECODE_STAGES * 2 * TILE_ELEMS * sizeof(bf16);
    const size_t merge = (size_t)(4 * 16 * D + 4 * 16 * 2 + 3 * 16 * MAX_SPLITS) * sizeof(float);
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(flash_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nsplit, Hkv, n_items);
    kvb_launch(flash_decode_kernel, dim3(grid), dim3(128), smem, stream, p);
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Decode with the splits of one (item, kv head) as a thread-block cluster: the same scan as above, but the
// splits meet through distributed shared memory.  Each block leaves its (m, l, acc) in its own shared memory;
// after a cluster barrier block s merges rows s, s + nsplit, ... from all blocks, in split order, and stores
// them.  No scratch in global memory, no counter, no block that is left alone with the merge.
//
// Keys and values that earlier steps wrote do not depend on the kernel before this one in the stream, so the
// step's segment data, the block table and the first tiles are fetched before the wait on that kernel; only
// the queries, and tiles that hold this step's own keys, are read after it.
// ---------------------------------------------------------------------------------------------
// Stages of keys/values in shared memory: two blocks share an SM.  (A block that takes most of an SM's shared
// memory to request its whole split at once was measured slower: clusters of such blocks wait long for a place.)
// For head sizes up to 64 a stage holds two 64-key tiles and a warp takes 32 keys of it: half as many barriers
// per key, and four independent chains of MMAs instead of two.
#define CLUSTER_STAGES 3
#define CLUSTER_KW (KVB_HEAD_DIM <= 64 ? 2 : 1)      // key tiles per stage
constexpr int MAX_CLUSTER = 8;      // the portable limit; clusters of 16 were measured slower (they wait long for a place)

template <int STAGES, int KW>
__global__ void __launch_bounds__(128) flash_decode_cluster_kernel(const __grid_constant__ DecodeParams p) {
    TRACE(0)
#ifdef KVB_TRACE
    if (threadIdx.x == 0) { unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid)); const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x; if (cta < 8192) kvb_trace_buf[cta * 8 + 7] = smid; }
#endif
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    const int split = blockIdx.x, hk = blockIdx.y, item = blockIdx.z;       // the cluster spans x: split is the rank
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = p.Hq / p.Hkv;
    // Written by the host's copy at the start of the step: safe to read before the wait.
    const int seg = p.items ? p.items[item] : item;
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int rows = min(q_len * G, 16);   // an item is one warp tile of 16 rows; rows beyond it are not this kernel's (see no_alloc.h)
    const int first_pos = kv_len - q_len;
    const int key_lo = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
    const int tile_begin = key_lo / KT, tile_end = (kv_len + KT - 1) / KT;
    const int num_tiles = tile_end - tile_begin;
    // A stage holds KW key tiles, of which each warp takes 16 * KW keys; a split is a whole number of stages.
    const int per_split = ((num_tiles + p.nsplit - 1) / p.nsplit + KW - 1) / KW * KW;
    const int my_begin = tile_begin + split * per_split;
    const int my_end = min(tile_end, my_begin + per_split);
    const int n = max(0, (my_end - my_begin + KW - 1) / KW);                // stages to scan; a split may be empty and still joins the barriers
    constexpr int NK = 16 * KW, STAGE_ELEMS = 2 * KW * TILE_ELEMS;

    KVSource src{p.k_pages, p.v_pages, p.block_table + (size_t)seg * p.table_stride, hk, p.Hkv, p.page_size, p.page_shift};
    auto load_stage = [&](int i) {                                          // key tiles my_begin + i KW .. + KW - 1; beyond kv_len: zeros
        bf16* ks = smem + (i % STAGES) * STAGE_ELEMS;
#pragma unroll
        for (int h = 0; h < KW; ++h)
            load_tile(ks + h * TILE_ELEMS, ks + (KW + h) * TILE_ELEMS, src, (my_begin + i * KW + h) * KT, key_lo, kv_len);
    };
    // The stages of the prologue are old if all their keys lie before this step's first position.
    const bool early = (my_begin + min(n, STAGES - 1) * KW) * KT <= first_pos;
    if (early) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < n) load_stage(s);
            cp_async_commit();
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    TRACE(1)
    if (!early) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < n) load_stage(s);
            cp_async_commit();
        }
    }
    WarpRows w;
    rows_init(w);
    auto q_row = [&](int r) -> const bf16* {
        return r < rows ? p.q + ((size_t)(q_start + r / G) * p.Hq + hk * G + r % G) * D : nullptr;
    };
    rows_load_q(w, q_row);
    w.pos[0] = g < rows ? first_pos + g / G : -1;
    w.pos[1] = g + 8 < rows ? first_pos + (g + 8) / G : -1;

    for (int i = 0; i < n; ++i) {
        if (i + STAGES - 1 < n) load_stage(i + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (i == 0) { TRACE(2) }
        const bf16* ks = smem + (i % STAGES) * STAGE_ELEMS;
        const int key0 = (my_begin + i * KW) * KT + warp * NK;
        if (key0 < kv_len)
            rows_tile_auto<NK>(w, ks + warp * NK * STRIDE, ks + KW * TILE_ELEMS + warp * NK * STRIDE, key0, p.window,
                               p.scale_log2, first_pos, kv_len - 1, true);
        __syncthreads();
    }
    cp_async_wait<0>();
    rows_finish_sum(w);
    TRACE(3)

    // The four warps' results meet in shared memory (the stages are free now), then the block's own result.
    float* wo = reinterpret_cast<float*>(smem_raw);            // [4][16][D]
    float* wml = wo + 4 * 16 * D;                              // [4][16][2]
    float* res_o = wml + 4 * 16 * 2;                           // [16][D]   this block's acc
    float* res_ml = res_o + 16 * D;                            // [16][2]   this block's (m, l)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int i = 0; i < NT_O; ++i)
            *reinterpret_cast<float2*>(wo + (warp * 16 + row) * D + i * 8 + 2 * t) = make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
        if (t == 0) { wml[(warp * 16 + row) * 2] = w.m[r]; wml[(warp * 16 + row) * 2 + 1] = w.l[r]; }
    }
    __syncthreads();
    for (int idx = tid; idx < rows * D; idx += 128) {
        const int row = idx / D, d = idx - row * D;
        float M = NEG_INF;
#pragma unroll
        for (int x = 0; x < 4; ++x) M = fmaxf(M, wml[(x * 16 + row) * 2]);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const float e = exp2f(wml[(x * 16 + row) * 2] - base);
            L += e * wml[(x * 16 + row) * 2 + 1];
            acc += e * wo[(x * 16 + row) * D + d];
        }
        if (p.nsplit == 1) {
            p.out[((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            res_o[row * D + d] = acc;
            if (d == 0) { res_ml[row * 2] = M; res_ml[row * 2 + 1] = L; }
        }
    }
    if (p.nsplit == 1) return;

    cluster_sync_all();                                        // every block's result is in its shared memory
    TRACE(4)
    // Block s takes rows s, s + nsplit, ...; a thread takes four columns of one row.
    // weight_s = 2^(m_s - M) / sum_s 2^(m_s - M) l_s; out = sum_s weight_s acc_s, added in split order.
    const int my_rows = rows > split ? (rows - split + p.nsplit - 1) / p.nsplit : 0;
    for (int idx = tid; idx < my_rows * (D / 4); idx += 128) {
        const int row = split + (idx / (D / 4)) * p.nsplit, d = (idx % (D / 4)) * 4;
        float2 ml[MAX_CLUSTER];
        float4 v[MAX_CLUSTER];
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            if (s < p.nsplit) {
                ml[s] = peer_ld2(peer_smem(res_ml + row * 2, s));
                v[s] = peer_ld4(peer_smem(res_o + row * D + d, s));
            } else {
                ml[s] = make_float2(NEG_INF, 0.f);
                v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float M = NEG_INF;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) M = fmaxf(M, ml[s].x);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f;
        float e[MAX_CLUSTER];
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            e[s] = exp2f(ml[s].x - base);
            L += e[s] * ml[s].y;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            const float ws = e[s] * inv;
            acc.x += ws * v[s].x; acc.y += ws * v[s].y; acc.z += ws * v[s].z; acc.w += ws * v[s].w;
        }
        bf16* o = p.out + ((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d;
        *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
    TRACE(5)
    cluster_sync_all();                                        // no block leaves while another still reads its result
    TRACE(6)
}

// The splits as a cluster: nsplit 1..8, no scratch.
KVB_API int kvb_flash_decode_cluster(const void* q, void* out, const void* k_pages, const void* v_pages,
                                     const int* block_table, int table_stride, const int* items, int n_items,
                                     const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, int Hq, int Hkv,
                                     int page_size, int window, int nsplit, float scale, cudaStream_t stream) {
    if (n_items <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (nsplit < 1 || nsplit > MAX_CLUSTER || n_items > 65535 || Hkv > 65535) return KVB_ERR_LIMIT;
    DecodeParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.items = items; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len;
    p.part_o = nullptr; p.part_ml = nullptr; p.tickets = nullptr;
    p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.nsplit = nsplit;
    p.scale_log2 = scale * 1.4426950408889634f;
    auto kernel = flash_decode_cluster_kernel<CLUSTER_STAGES, CLUSTER_KW>;
    size_t smem = (size_t)CLUSTER_STAGES * 2 * CLUSTER_KW * TILE_ELEMS * sizeof(bf16);
    const size_t merge = (size_t)(5 * 16 * D + 5 * 16 * 2) * sizeof(float);
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nsplit, Hkv, n_items);
    kvb_launch_cluster(kernel, dim3(grid), dim3(128), (unsigned)nsplit, smem, stream, p);
    return kvb_launch_status();
}

#if KVB_HEAD_DIM % 64 == 0
// ---------------------------------------------------------------------------------------------
// The cluster kernel with keys and values brought by TMA (head sizes 64 and 128, pages of 8..64 tokens): a fifth
// warp looks pages up and issues one tiled copy per page and 64 columns - a few large requests instead of
// thousands of 16-byte ones - into 128-byte-swizzled stages; a stage is handed to the four scanning warps
// through a "full" mbarrier and handed back through an "empty" one.  Everything else - the split into a
// cluster, the merge, what is fetched before the wait - is as above.  Waits are bounded: on a timeout the
// error word is set and the block winds down (it still joins the cluster's barriers).
// ---------------------------------------------------------------------------------------------
namespace dtma {
using namespace tc;
constexpr int HALVES = D / 64;
constexpr int KW = D == 64 ? 2 : 1;                       // 64-key tiles per stage
constexpr int MAX_STAGES = 4;                             // a ring of three stages, or of four where a block has an SM to itself
constexpr int NKEYS = 64 * KW;
constexpr int HALF_BYTES = NKEYS * 128;                   // a [NKEYS x 64 columns] swizzled sub-tile
constexpr int KV_BYTES = HALVES * HALF_BYTES;             // keys of a stage; values follow
constexpr int STAGE_BYTES = 2 * KV_BYTES;
constexpr int RECV_BYTES = 24 * (D + 2) * 4;               // nsplit * ceil(16 / nsplit) <= 24 row slots of (m, l, acc)
constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + RECV_BYTES + 1024; }

struct Shared {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES];
    int failed;
};

// FUSED: the step's rows come straight from the q/k/v product (every segment brings one token).  The kernel adds the
// biases and rotates the queries itself, and the block whose keys include the new position also makes the new key and
// value (src/qwen_kernels.cu:45-53 and :63-79 of the reference, folded into its attention): it writes them into their
// page and into the stage of shared memory that the copy of that page has filled, since the copy ran before they existed.
struct NewRows {
    const bf16* qkv;           // [T, (Hq + 2 Hkv) D]: queries, keys, values of each row
    const float* bias;         // [(Hq + 2 Hkv) D] or nullptr
    const float* cos_t;        // [table_len, rot_half]; rot_half 0: no rotation
    const float* sin_t;
    bf16* k_pages;
    bf16* v_pages;
    int rot_half, table_len;
};

// N elements of a row of the q/k/v product with their biases, rotated by the angles of a position.  What does not
// depend on the product - the biases and the angles - is fetched by `prepare`, before the wait for the product; `finish`
// then reads the elements and their rotation partners.  No load sits behind a branch (where a table does not apply the
// load goes to a valid address and its value is dropped), so each of the two costs one trip to memory.
template <int N>
struct NewElements {
    int idx[N], pidx[N];
    float bx[N], bp[N], c[N], sn[N];
    bool rot[N], low[N];
    __device__ __forceinline__ void prepare(const NewRows& nr, const int (&head)[N], const int (&d)[N], int pos, bool rotate) {
        const float* spare = reinterpret_cast<const float*>(nr.qkv);      // any address that can be read
#pragma unroll
        for (int j = 0; j < N; ++j) {
            idx[j] = head[j] * D + d[j];
            rot[j] = rotate && d[j] < 2 * nr.rot_half;
            low[j] = d[j] < nr.rot_half;
            pidx[j] = rot[j] ? (low[j] ? idx[j] + nr.rot_half : idx[j] - nr.rot_half) : idx[j];
            const int t0 = low[j] ? d[j] : d[j] - nr.rot_half;
            bx[j] = *(nr.bias ? nr.bias + idx[j] : spare);
            bp[j] = *(nr.bias ? nr.bias + pidx[j] : spare);
            c[j] = *(rot[j] ? nr.cos_t + (size_t)pos * nr.rot_half + t0 : spare);
            sn[j] = *(rot[j] ? nr.sin_t + (size_t)pos * nr.rot_half + t0 : spare);
        }
    }
    __device__ __forceinline__ void finish(const NewRows& nr, const bf16* row, float (&out)[N]) const {
        bf16 xr[N], pr[N];
#pragma unroll
        for (int j = 0; j < N; ++j) { xr[j] = row[idx[j]]; pr[j] = row[pidx[j]]; }
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const float x = __bfloat162float(xr[j]) + (nr.bias ? bx[j] : 0.f);
            const float xp = __bfloat162float(pr[j]) + (nr.bias ? bp[j] : 0.f);
            out[j] = !rot[j] ? x : (low[j] ? (x * c[j] - xp * sn[j]) : (x * c[j] + xp * sn[j]));
        }
    }
};

template <bool FUSED, int STAGES>
__global__ void __launch_bounds__(160) flash_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                               const __grid_constant__ CUtensorMap map_v,
                                                               const __grid_constant__ DecodeParams p,
                                                               const __grid_constant__ NewRows nr, int* err) {
    TRACE(0)
    if (p.nsplit > 1) cluster_arrive_started();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ Shared sh;
    // The cluster spans x: split is the rank.  With several clusters per (item, kv head), y counts (kv head, cluster)
    // and the keys are cut into nsuper * nsplit runs, cluster c taking runs c nsplit .. c nsplit + nsplit - 1.
    const int split = blockIdx.x, hk = blockIdx.y / p.nsuper, super = blockIdx.y - hk * p.nsuper, item = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = p.Hq / p.Hkv;
    // Written by the host's copy at the start of the step: safe to read before the wait.
    const int seg = p.items ? p.items[item] : item;
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int rows = min(q_len * G, 16);   // an item is one warp tile of 16 rows; rows beyond it are not this kernel's (see no_alloc.h)
    const int first_pos = kv_len - q_len;
    const int key_lo = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
    const int tile_begin = key_lo / KT, tile_end = (kv_len + KT - 1) / KT;
    const int num_tiles = tile_end - tile_begin;
    const int runs = p.nsplit * p.nsuper;
    const int per_split = ((num_tiles + runs - 1) / runs + KW - 1) / KW * KW;
    const int my_begin = min(tile_end, tile_begin + (super * p.nsplit + split) * per_split);
    const int my_end = min(tile_end, my_begin + per_split);
    const int n = max(0, (my_end - my_begin + KW - 1) / KW);                // stages to scan

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 4); }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    WarpRows w;
    rows_init(w);
    if (warp == 4) {
        // ---- loader warp ----
        const int* table = p.block_table + (size_t)seg * p.table_stride;
        const int pages_per_stage = NKEYS >> p.page_shift;
        bool ok = true;
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
        }
        // Stage i holds keys [(my_begin + i KW) * 64, + NKEYS).  Lane pg takes page pg of it: its number is looked up ahead
        // of the copy (the ring's first round all at once, then one stage ahead), so that the table's latency is paid
        // once and not stage by stage.  -1: beyond the last key, or given back behind a window.
        auto lookup = [&](int i) -> int {
            int page = -1;
            if (lane < pages_per_stage && i < n) {
                const int first_key = (my_begin + i * KW) * KT + lane * p.page_size;
                if (first_key < kv_len && first_key + p.page_size > key_lo) page = table[first_key >> p.page_shift];
            }
            return page;
        };
        // Every lane asks the barrier (one lane asking and telling the others costs twice as much).  A page that is not
        // there is copied from before the pool's first row: the TMA unit fills what lies outside the tensor with zeros
        // (the slot must hold finite numbers, because 0 * NaN would poison the sums) and still counts the bytes.
        auto load_stage = [&](int i, int my_page) {
            const int s = i % STAGES;
            unsigned char* dst = stages + (size_t)s * STAGE_BYTES;
            if (i >= STAGES) {
                ok = mbar_wait(&sh.empty[s], ((i - STAGES) / STAGES) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return;
            }
            if (lane == 0) mbar_expect_tx(&sh.full[s], (uint32_t)pages_per_stage * 2 * HALVES * p.page_size * 128);
            __syncwarp();
            if (lane < pages_per_stage) {
                const int row = my_page >= 0 ? (my_page * p.Hkv + hk) * p.page_size : -p.page_size;   // of the pool as [pages * heads * page, D]
#pragma unroll
                for (int hb = 0; hb < HALVES; ++hb) {
                    tma_load_2d(dst + hb * HALF_BYTES + lane * p.page_size * 128, &map_k, hb * 64, row, &sh.full[s]);
                    tma_load_2d(dst + KV_BYTES + hb * HALF_BYTES + lane * p.page_size * 128, &map_v, hb * 64, row, &sh.full[s]);
                }
            }
        };
        // A stage is old if all its keys lie before this step's first position: the old ones among the ring's first
        // round are fetched before the wait.  Fused, all of them are old: nobody but this kernel writes the pool
        // meanwhile, and the new position's slot is made afresh in shared memory.
        const int first = min(n, STAGES);
        int first_pages[STAGES];
#pragma unroll
        for (int i = 0; i < STAGES; ++i) first_pages[i] = lookup(i);
        int page_next = lookup(STAGES);
        unsigned early = 0;
#pragma unroll
        for (int i = 0; i < STAGES; ++i)
            if (i < first && (FUSED || (my_begin + (i + 1) * KW) * KT <= first_pos)) { load_stage(i, first_pages[i]); early |= 1u << i; }
        pdl_wait();
        pdl_launch_dependents();
#pragma unroll
        for (int i = 0; i < STAGES; ++i)
            if (i < first && !((early >> i) & 1u)) load_stage(i, first_pages[i]);
        for (int i = first; i < n && ok; ++i) {
            const int page = page_next;
            page_next = lookup(i + 1);
            load_stage(i, page);
        }
        if (!ok && lane == 0) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; }
    } else {
        // ---- scanning warps ----
        __shared__ __align__(16) unsigned short new_q_raw[FUSED ? 16 * D : 8];
        bf16* new_q = reinterpret_cast<bf16*>(new_q_raw);
        const int width = (p.Hq + 2 * p.Hkv) * D;
        // Fused: the warp whose keys of stage `new_stage` include the new position makes the new key and value.  It
        // fetches them, like every warp its share of the queries, in one round of loads right after the wait.
        constexpr int NK = 16 * KW;
        constexpr int PER_LANE = D / 32;
        int new_stage = -1, new_page = -1;
        float kn[PER_LANE], vn[PER_LANE];
        if (FUSED) {
            const int tile = first_pos / KT;
            if (tile >= my_begin && tile < my_end) {
                const int i = (tile - my_begin) / KW;
                if ((first_pos - (my_begin + i * KW) * KT) / NK == warp) {
                    new_stage = i;
                    new_page = p.block_table[(size_t)seg * p.table_stride + (first_pos >> p.page_shift)];
                }
            }
        }
        // One token a segment: row r is query head hk G + r at the position of the new key.  A thread makes elements
        // tid, tid + 128, ... of the rows' rows * D (the first QN of them prepared ahead; indices beyond the rows are
        // clamped: loaded, not stored).
        constexpr int QN = 4;
        NewElements<QN> qe;
        NewElements<PER_LANE> ke, ve;
        const bool pos_ok = !FUSED || nr.rot_half == 0 || first_pos < nr.table_len;
        const int pos = pos_ok ? first_pos : 0;
        if (FUSED) {
            int head[QN], d[QN];
#pragma unroll
            for (int j = 0; j < QN; ++j) {
                const int idx = min(128 * j + tid, rows * D - 1);
                head[j] = hk * G + idx / D;
                d[j] = idx % D;
            }
            qe.prepare(nr, head, d, pos, true);
            if (new_stage >= 0) {
                int khead[PER_LANE], vhead[PER_LANE], dd[PER_LANE];
#pragma unroll
                for (int j = 0; j < PER_LANE; ++j) { khead[j] = p.Hq + hk; vhead[j] = p.Hq + p.Hkv + hk; dd[j] = lane + 32 * j; }
                ke.prepare(nr, khead, dd, pos, true);
                ve.prepare(nr, vhead, dd, pos, false);                            // values are not rotated
            }
        }
        pdl_wait();
        pdl_launch_dependents();
        TRACE(1)
        if (FUSED) {
            if (!pos_ok && tid == 0) atomicOr(err, KVB_DEV_BAD_POS);
            const bf16* src = nr.qkv + (size_t)q_start * width;
            if (new_stage >= 0) {
                if (new_page < 0 && lane == 0) atomicOr(err, KVB_DEV_BAD_PAGE);
                ke.finish(nr, src, kn);
                ve.finish(nr, src, vn);
            }
            float x[QN];
            qe.finish(nr, src, x);
#pragma unroll
            for (int j = 0; j < QN; ++j) {
                const int idx = 128 * j + tid;
                if (idx < rows * D) new_q[idx] = __float2bfloat16_rn(x[j]);
            }
            for (int base = 128 * QN; base < rows * D; base += 128 * QN) {       // more rows than the usual groups have
                int head[QN], d[QN];
#pragma unroll
                for (int j = 0; j < QN; ++j) {
                    const int idx = min(base + 128 * j + tid, rows * D - 1);
                    head[j] = hk * G + idx / D;
                    d[j] = idx % D;
                }
                NewElements<QN> more;
                more.prepare(nr, head, d, pos, true);
                more.finish(nr, src, x);
#pragma unroll
                for (int j = 0; j < QN; ++j) {
                    const int idx = base + 128 * j + tid;
                    if (idx < rows * D) new_q[idx] = __float2bfloat16_rn(x[j]);
                }
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");          // the four scanning warps
            TRACE(6)
        }
        auto q_row = [&](int r) -> const bf16* {
            if (FUSED) return r < rows ? new_q + r * D : nullptr;
            return r < rows ? p.q + ((size_t)(q_start + r / G) * p.Hq + hk * G + r % G) * D : nullptr;
        };
        rows_load_q(w, q_row);
        w.pos[0] = g < rows ? first_pos + g / G : -1;
        w.pos[1] = g + 8 < rows ? first_pos + (g + 8) / G : -1;
        for (int i = 0; i < n; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(&sh.full[s], (i / STAGES) & 1)) {
                if (lane == 0) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; }
                break;
            }
            if (i == 0) { TRACE(2) }
            unsigned char* base = stages + (size_t)s * STAGE_BYTES + warp * NK * 128;   // this warp's keys: rows warp NK ..
            const int key0 = (my_begin + i * KW) * KT + warp * NK;
            if (FUSED && i == new_stage) {
                // Into their page, and over what the copy left at their row.
                const size_t at = ((size_t)max(new_page, 0) * p.Hkv + hk) * p.page_size * D + (size_t)(first_pos & (p.page_size - 1)) * D;
                const int row = first_pos - key0;
                const SwizzledTile kt{base, HALF_BYTES}, vt{base + KV_BYTES, HALF_BYTES};
#pragma unroll
                for (int j = 0; j < PER_LANE; ++j) {
                    const int d = lane + 32 * j;
                    const bf16 kb = __float2bfloat16_rn(kn[j]), vb = __float2bfloat16_rn(vn[j]);
                    const_cast<bf16*>(kt.at(row, d & ~7))[d & 7] = kb;
                    const_cast<bf16*>(vt.at(row, d & ~7))[d & 7] = vb;
                    if (new_page >= 0) { nr.k_pages[at + d] = kb; nr.v_pages[at + d] = vb; }
                }
                __syncwarp();
            }
            if (key0 < kv_len)
                rows_tile_auto_in<NK>(w, SwizzledTile{base, HALF_BYTES}, SwizzledTile{base + KV_BYTES, HALF_BYTES}, key0,
                                      p.window, p.scale_log2, first_pos, kv_len - 1, true);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty[s]);
        }
        rows_finish_sum(w);
        TRACE(3)
    }
    __syncthreads();                                           // every stage has been read: the merge may reuse them

    float* wo = reinterpret_cast<float*>(stages);              // [4][16][D]
    float* wml = wo + 4 * 16 * D;                              // [4][16][2]
    // What the other blocks of the cluster send: slot s holds block s's (m, l, acc) of the rows this block finishes
    // (rows split, split + nsplit, ...: at most `rpo` of them).  It lies behind the stages, which a block may
    // still be filling while others already send.
    const int rpo = (16 + p.nsplit - 1) / p.nsplit;
    float* recv_o = reinterpret_cast<float*>(stages + STAGES * STAGE_BYTES);   // [nsplit][rpo][D]
    float* recv_ml = recv_o + p.nsplit * rpo * D;                                // [nsplit][rpo][2]
    if (warp < 4) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<float2*>(wo + (warp * 16 + row) * D + i * 8 + 2 * t) = make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
            if (t == 0) { wml[(warp * 16 + row) * 2] = w.m[r]; wml[(warp * 16 + row) * 2 + 1] = w.l[r]; }
        }
    }
    __syncthreads();
    if (p.nsplit > 1) cluster_wait_started();                  // every block of the cluster is running: its memory may be written
    // The four warps' results become the block's: four columns of one row per thread and step.
    for (int idx = tid; idx < rows * (D / 4); idx += 160) {
        const int row = idx / (D / 4), d = (idx - row * (D / 4)) * 4;
        float M = NEG_INF;
#pragma unroll
        for (int x = 0; x < 4; ++x) M = fmaxf(M, wml[(x * 16 + row) * 2]);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const float e = exp2f(wml[(x * 16 + row) * 2] - base);
            const float4 v = *reinterpret_cast<const float4*>(wo + (x * 16 + row) * D + d);
            L += e * wml[(x * 16 + row) * 2 + 1];
            acc.x += e * v.x; acc.y += e * v.y; acc.z += e * v.z; acc.w += e * v.w;
        }
        if (p.nsplit == 1) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            bf16* o = p.out + ((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d;
            *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        } else {
            // To the block that finishes this row, into the slot of this split.
            const int owner = row % p.nsplit, k = row / p.nsplit;
            peer_st4(peer_smem(recv_o + ((size_t)split * rpo + k) * D + d, owner), acc);
            if (d == 0) peer_st2(peer_smem(recv_ml + ((size_t)split * rpo + k) * 2, owner), make_float2(M, L));
        }
    }
    if (p.nsplit == 1) return;

    cluster_sync_all();                                        // what was sent has arrived; nobody reads another block's memory after this
    TRACE(4)
    // weight_s = 2^(m_s - M) / sum_s 2^(m_s - M) l_s; out = sum_s weight_s acc_s, added in split order.
    const int my_rows = rows > split ? (rows - split + p.nsplit - 1) / p.nsplit : 0;
    for (int idx = tid; idx < my_rows * (D / 4); idx += 160) {
        const int k = idx / (D / 4), row = split + k * p.nsplit, d = (idx % (D / 4)) * 4;
        float2 ml[MAX_CLUSTER];
        float4 v[MAX_CLUSTER];
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            if (s < p.nsplit) {
                ml[s] = *reinterpret_cast<const float2*>(recv_ml + ((size_t)s * rpo + k) * 2);
                v[s] = *reinterpret_cast<const float4*>(recv_o + ((size_t)s * rpo + k) * D + d);
            } else {
                ml[s] = make_float2(NEG_INF, 0.f);
                v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float M = NEG_INF;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) M = fmaxf(M, ml[s].x);
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f;
        float e[MAX_CLUSTER];
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            e[s] = exp2f(ml[s].x - base);
            L += e[s] * ml[s].y;
        }
        const float inv = p.nsuper > 1 ? 1.f : (L > 0.f ? 1.f / L : 0.f);     // several clusters: the sums stay unscaled
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER; ++s) {
            const float ws = e[s] * inv;
            acc.x += ws * v[s].x; acc.y += ws * v[s].y; acc.z += ws * v[s].z; acc.w += ws * v[s].w;
        }
        if (p.nsuper > 1) {
            // This cluster's (m, l, acc) of the row, left for the cluster that finishes last.
            const size_t slot = (((size_t)item * p.Hkv + hk) * p.nsuper + super) * 16 + row;
            *reinterpret_cast<float4*>(p.part_o + slot * D + d) = acc;
            if (d == 0) *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(M, L);
        } else {
            bf16* o = p.out + ((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d;
            *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
        }
    }
    if (p.nsuper > 1) {
        // The clusters of an (item, kv head) meet through memory: each block counts in on the ticket of its rows
        // (rows split, split + nsplit, ...); the last one to arrive adds the clusters' sums in cluster order.
        __shared__ int last_s;
        __threadfence();
        __syncthreads();
        int* ticket = p.tickets + ((size_t)item * p.Hkv + hk) * p.nsplit + split;
        if (tid == 0) {
            last_s = atomicAdd(ticket, 1) == p.nsuper - 1;
            if (last_s) *ticket = 0;                                 // zero again for the next launch
        }
        __syncthreads();
        if (!last_s) return;
        __threadfence();
        for (int idx = tid; idx < my_rows * (D / 4); idx += 160) {
            const int k = idx / (D / 4), row = split + k * p.nsplit, d = (idx % (D / 4)) * 4;
            const size_t slot0 = (((size_t)item * p.Hkv + hk) * p.nsuper) * 16 + row;
            float M = NEG_INF;
            for (int c = 0; c < p.nsuper; ++c) M = fmaxf(M, __ldcg(p.part_ml + (slot0 + (size_t)c * 16) * 2));
            const float base = M == NEG_INF ? 0.f : M;
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = 0; c < p.nsuper; ++c) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (slot0 + (size_t)c * 16) * 2));
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + (slot0 + (size_t)c * 16) * D + d));
                const float e = exp2f(ml.x - base);
                L += e * ml.y;
                acc.x += e * v.x; acc.y += e * v.y; acc.z += e * v.z; acc.w += e * v.w;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            bf16* o = p.out + ((size_t)(q_start + row / G) * p.Hq + hk * G + row % G) * D + d;
            *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
    }
    TRACE(5)
}

// How many clusters of `nsplit` blocks of the TMA decode kernel the GPU holds at once (0 on an error): a grid with more
// clusters than that runs in waves, which costs a whole kernel's latency again.
template <int STAGES>
static int max_clusters(int nsplit) {
    if (cudaFuncSetAttribute(flash_decode_tma_kernel<true, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(STAGES)) != cudaSuccess) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(nsplit * 64);
    config.blockDim = dim3(160);
    config.dynamicSmemBytes = smem_bytes(STAGES);
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = nsplit;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, flash_decode_tma_kernel<true, STAGES>, &config) != cudaSuccess) return 0;
    return clusters;
}
}  // namespace dtma

KVB_API int kvb_flash_decode_tma_max_clusters(int nsplit) {
    if (nsplit < 1 || nsplit > MAX_CLUSTER) return 0;
    return dtma::max_clusters<3>(nsplit);
}

// The splits as a cluster, keys and values by TMA: nsplit 1..8, page_size a power of two 8..64, num_pages the pool's
// page count, err the device error word.  With `qkv` (then `q` is not read, `items` must be null and every segment
// bring one token) the kernel takes the rows of the q/k/v product instead of rotated queries and appended keys:
// bias [(Hq + 2 Hkv) D] or null, cos_t / sin_t [table_len, rot_half] (rot_half 0: no rotation).
// Where the grid's clusters all fit with one block on an SM, the blocks take a ring of four stages instead of three:
// at 4,096 tokens over eight splits that is a block's whole share, all of it requested before the wait.
KVB_API int kvb_flash_decode_tma(const void* q, void* out, void* k_pages, void* v_pages, int num_pages,
                                 const int* block_table, int table_stride, const int* items, int n_items,
                                 const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, int Hq, int Hkv,
                                 int page_size, int window, int nsplit, float scale, const void* qkv, const float* bias,
                                 const float* cos_t, const float* sin_t, int rot_half, int table_len, int nsuper,
                                 float* scratch, int* tickets, int* err, cudaStream_t stream) {
    using namespace dtma;
    if (n_items <= 0) return KVB_OK;
    // Several clusters per (item, kv head): `scratch` holds n_items * Hkv * nsuper * 16 * (D + 2) floats, `tickets`
    // n_items * Hkv * nsplit ints that are zero before the first launch (the kernel leaves them zero).
    if (nsuper < 1 || nsuper > 64 || (nsuper > 1 && (nsplit < 2 || qkv || !scratch || !tickets))) return KVB_ERR_SHAPE;
    if ((long long)Hkv * nsuper > 65535) return KVB_ERR_LIMIT;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return KVB_ERR_SHAPE;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (nsplit < 1 || nsplit > MAX_CLUSTER || n_items > 65535 || Hkv > 65535) return KVB_ERR_LIMIT;
    if (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return KVB_ERR_ALIGN;
    if (qkv && (items != nullptr || rot_half < 0 || 2 * rot_half > D || (rot_half > 0 && (!cos_t || !sin_t)))) return KVB_ERR_SHAPE;
    CUtensorMap mk, mv;
    const long long pool_rows = (long long)num_pages * Hkv * page_size;
    int rc = make_bf16_map(&mk, k_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    rc = make_bf16_map(&mv, v_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    DecodeParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.items = items; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len;
    p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)n_items * Hkv * nsuper * 16 * D : nullptr; p.tickets = tickets;
    p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window; p.nsplit = nsplit; p.nsuper = nsuper;
    p.scale_log2 = scale * 1.4426950408889634f;
    NewRows nr{(const bf16*)qkv, bias, cos_t, sin_t, (bf16*)k_pages, (bf16*)v_pages, rot_half, table_len};
    static bool configured = false;
    static int deep_clusters[MAX_CLUSTER + 1];                 // clusters of each size that fit with the ring of four
    if (!configured) {
        const void* kernels[4] = {(const void*)flash_decode_tma_kernel<false, 3>, (const void*)flash_decode_tma_kernel<true, 3>,
                                  (const void*)flash_decode_tma_kernel<false, 4>, (const void*)flash_decode_tma_kernel<true, 4>};
        for (int i = 0; i < 4; ++i) {
            cudaError_t e = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(i < 2 ? 3 : 4));
            if (e != cudaSuccess) return (int)e;
            e = cudaFuncSetAttribute(kernels[i], cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return (int)e;
        }
        for (int c = 1; c <= MAX_CLUSTER; ++c) deep_clusters[c] = max_clusters<4>(c);
        configured = true;
    }
    dim3 grid(nsplit, Hkv * nsuper, n_items);
    const bool deep = (long long)n_items * Hkv * nsuper <= deep_clusters[nsplit];
    if (qkv && deep)
        kvb_launch_cluster(flash_decode_tma_kernel<true, 4>, dim3(grid), dim3(160), (unsigned)nsplit, (size_t)smem_bytes(4), stream, mk, mv, p, nr, err);
    else if (qkv)
        kvb_launch_cluster(flash_decode_tma_kernel<true, 3>, dim3(grid), dim3(160), (unsigned)nsplit, (size_t)smem_bytes(3), stream, mk, mv, p, nr, err);
    else if (deep)
        kvb_launch_cluster(flash_decode_tma_kernel<false, 4>, dim3(grid), dim3(160), (unsigned)nsplit, (size_t)smem_bytes(4), stream, mk, mv, p, nr, err);
    else
        kvb_launch_cluster(flash_decode_tma_kernel<false, 3>, dim3(grid), dim3(160), (unsigned)nsplit, (size_t)smem_bytes(3), stream, mk, mv, p, nr, err);
    return kvb_launch_status();
}
#endif

// ---------------------------------------------------------------------------------------------
// Prefill: one block of four warps per (unit, query head).  A tile is 64 consecutive query positions of one
// segment (16 per warp); its keys run from the first key its first row sees to its last row's own position.
// Causal tiles differ in length by a factor of the sequence length over 64, so a tile is cut into units of a
// bounded number of key tiles (`nsplit` units; the host chooses it from the tile's length): units are what the
// grid is made of, and they are all about the same size.  A tile with one unit stores its rows directly;
// otherwise each unit leaves (m, l, acc) of its rows in scratch and the last unit of a (tile, head) to finish
// (a ticket counter) merges them in unit order, as the decode kernel does with its splits.
// A warp skips key tiles that none of its rows see.
// ---------------------------------------------------------------------------------------------
struct PrefillParams {
    const bf16* q;
    bf16* out;
    const bf16* k_pages;
    const bf16* v_pages;
    const int* block_table;
    const int* units;          // [n_units, 8]: segment, first row of the tile, unit, units of the tile, tile id, index of the tile's first unit
    const int* seg_q_start;
    const int* seg_q_len;
    const int* seg_kv_len;
    float* part_o;             // [n_units, Hq, 64, D]
    float* part_ml;            // [n_units, Hq, 64, 2]
    int* tickets;              // [n_tiles, Hq], zero between launches
    int table_stride, Hq, Hkv, page_size, page_shift, window;
    float scale_log2;
};

__global__ void __launch_bounds__(128) flash_prefill_kernel(const PrefillParams p) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int ticket_s;
    const int unit = blockIdx.x, h = blockIdx.y;
    const int* u = p.units + 8 * unit;
    const int seg = u[0], row0 = u[1], split = u[2], nsplit = u[3], tile_id = u[4], unit0 = u[5];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int hk = h / (p.Hq / p.Hkv);
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int first_pos = kv_len - q_len;                    // position of the segment's first row
    const int tile_rows = min(64, q_len - row0);
    const int pos_first = first_pos + row0, pos_last = first_pos + row0 + tile_rows - 1;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int tile_begin = key_lo / KT, tile_end = pos_last / KT + 1;
    const int num_tiles = tile_end - tile_begin;
    const int per_split = (num_tiles + nsplit - 1) / nsplit;
    const int n_valid = (num_tiles + per_split - 1) / per_split;   // units of this tile that have keys (a window may leave fewer)
    if (split >= n_valid) return;
    const int kt_begin = tile_begin + split * per_split;
    const int kt_end = min(tile_end, kt_begin + per_split);
    const int n = kt_end - kt_begin;

    KVSource src{p.k_pages, p.v_pages, p.block_table + (size_t)seg * p.table_stride, hk, p.Hkv, p.page_size, p.page_shift};
    WarpRows w;
    rows_init(w);
    const int wrow0 = row0 + warp * 16;                       // this warp's first row within the segment
    auto q_row = [&](int r) -> const bf16* {
        return wrow0 + r < q_len ? p.q + ((size_t)(q_start + wrow0 + r) * p.Hq + h) * D : nullptr;
    };
    rows_load_q(w, q_row);
    w.pos[0] = wrow0 + g < q_len ? first_pos + wrow0 + g : -1;
    w.pos[1] = wrow0 + g + 8 < q_len ? first_pos + wrow0 + g + 8 : -1;
    const int warp_rows = min(16, q_len - wrow0);             // <= 0: the warp has no rows
    const int warp_pos_first = first_pos + wrow0, warp_pos_last = first_pos + wrow0 + warp_rows - 1;
    const int warp_key_lo = (p.window > 0 && warp_pos_first - p.window + 1 > 0) ? warp_pos_first - p.window + 1 : 0;

    constexpr int STAGES = PREFILL_STAGES;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n) load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (kt_begin + s) * KT, key_lo, pos_last + 1);
        cp_async_commit();
    }
    for (int i = 0; i < n; ++i) {
        const int ahead = i + STAGES - 1;
        if (ahead < n) {
            const int s = ahead % STAGES;
            load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (kt_begin + ahead) * KT, key_lo, pos_last + 1);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const int s = i % STAGES;
        const int key0 = (kt_begin + i) * KT;
        if (warp_rows > 0 && key0 <= warp_pos_last && key0 + KT > warp_key_lo)
            rows_tile_auto<KT>(w, smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, key0, p.window, p.scale_log2,
                               warp_pos_first, warp_pos_last, warp_rows == 16);
        __syncthreads();
    }
    rows_finish_sum(w);
    auto out_row = [&](int r) -> bf16* {
        return wrow0 + r < q_len ? p.out + ((size_t)(q_start + wrow0 + r) * p.Hq + h) * D : nullptr;
    };
    if (n_valid == 1) {
        rows_store(w, out_row);
        return;
    }
    // Leave this unit's (m, l, acc) for its 64 rows, then take a ticket.
    {
        float* po = p.part_o + ((size_t)(unit0 + split) * p.Hq + h) * 64 * D;
        float* pml = p.part_ml + ((size_t)(unit0 + split) * p.Hq + h) * 64 * 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = warp * 16 + g + 8 * r;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<float2*>(po + row * D + i * 8 + 2 * t) = make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
            if (t == 0) *reinterpret_cast<float2*>(pml + row * 2) = make_float2(w.m[r], w.l[r]);
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket_s = atomicAdd(p.tickets + tile_id * p.Hq + h, 1);
    __syncthreads();
    if (ticket_s != n_valid - 1) return;
    __threadfence();
    if (tid == 0) p.tickets[tile_id * p.Hq + h] = 0;
    // Merge in unit order.  weight[row][s] = 2^(m_s - M) / sum_s 2^(m_s - M) l_s; out = sum_s weight_s acc_s.
    float* wgt = reinterpret_cast<float*>(smem_raw);           // [64][PREFILL_MAX_UNITS]
    if (tid < tile_rows) {
        const int row = tid;
        float M = NEG_INF;
        float ms[PREFILL_MAX_UNITS], ls[PREFILL_MAX_UNITS];
#pragma unroll
        for (int s = 0; s < PREFILL_MAX_UNITS; ++s) {
            if (s < n_valid) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (((size_t)(unit0 + s) * p.Hq + h) * 64 + row) * 2));
                ms[s] = ml.x; ls[s] = ml.y;
            } else {
                ms[s] = NEG_INF; ls[s] = 0.f;
            }
            M = fmaxf(M, ms[s]);
        }
        const float base = M == NEG_INF ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (int s = 0; s < PREFILL_MAX_UNITS; ++s) {
            ms[s] = exp2f(ms[s] - base);
            L += ms[s] * ls[s];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int s = 0; s < PREFILL_MAX_UNITS; ++s) wgt[row * PREFILL_MAX_UNITS + s] = ms[s] * inv;
    }
    __syncthreads();
    for (int idx = tid; idx < tile_rows * (D / 4); idx += 128) {
        const int row = idx / (D / 4), d = (idx - row * (D / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < n_valid; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int x = 0; x < 8; ++x)
                v[x] = s0 + x < n_valid
                           ? __ldcg(reinterpret_cast<const float4*>(p.part_o + (((size_t)(unit0 + s0 + x) * p.Hq + h) * 64 + row) * D + d))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const float ws = s0 + x < n_valid ? wgt[row * PREFILL_MAX_UNITS + s0 + x] : 0.f;
                acc.x += ws * v[x].x; acc.y += ws * v[x].y; acc.z += ws * v[x].z; acc.w += ws * v[x].w;
            }
        }
        bf16* o = p.out + ((size_t)(q_start + row0 + row) * p.Hq + h) * D + d;
        *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
}

// `units`: int32 [n_units, 8] (see PrefillParams); `scratch`: n_units * Hq * 64 * (D + 2) floats (only read and
// written for tiles of more than one unit); `tickets`: n_tiles * Hq ints, zero before the first launch.
// A tile may have at most PREFILL_MAX_UNITS units.
KVB_API int kvb_flash_prefill_max_units() { return PREFILL_MAX_UNITS; }

KVB_API int kvb_flash_prefill(const void* q, void* out, const void* k_pages, const void* v_pages,
                              const int* block_table, int table_stride, const int* units, int n_units,
                              const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, float* scratch,
                              int* tickets, int Hq, int Hkv, int page_size, int window, float scale, cudaStream_t stream) {
    if (n_units <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (Hq > 65535) return KVB_ERR_LIMIT;
    PrefillParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.units = units; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)n_units * Hq * 64 * D;
    p.tickets = tickets;
    p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    size_t smem = (size_t)PREFILL_STAGES * 2 * TILE_ELEMS * sizeof(bf16);
    const size_t merge = (size_t)64 * PREFILL_MAX_UNITS * sizeof(float);
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_units, Hq);
    kvb_launch(flash_prefill_kernel, dim3(grid), dim3(128), smem, stream, p);
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate (see no_alloc.h).
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Scratch of kvb_flash_decode_static: partial results first, tickets in the last KVB_STATIC_TICKET_BYTES.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char kvb_static_scratch[KVB_STATIC_SCRATCH_BYTES];

int kvb_flash_decode_static(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                            int table_stride, const int* items, int n_items, const int* seg_q_start,
                            const int* seg_q_len, const int* seg_kv_len, int Hq, int Hkv, int page_size, int window,
                            int nsplit, float scale, cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static unsigned char* base_of_device[MAX_DEVICES] = {nullptr};
    if (n_items <= 0) return KVB_OK;
    // Everything the regular entry point would refuse is refused here first, before anything is queued on the stream.
    if (Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (nsplit < 1 || nsplit > MAX_SPLITS || n_items > 65535 || Hkv > 65535) return KVB_ERR_LIMIT;
    const size_t floats = (size_t)n_items * Hkv * nsplit * 16 * (D + 2);
    const size_t tickets = (size_t)n_items * Hkv;
    if (floats * sizeof(float) > KVB_STATIC_SCRATCH_BYTES - KVB_STATIC_TICKET_BYTES ||
        tickets * sizeof(int) > KVB_STATIC_TICKET_BYTES)
        return KVB_ERR_STATIC_SCRATCH;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) return KVB_ERR_LIMIT;
    if (!base_of_device[device]) {   // set-up, once per device, with that device current
        unsigned char* base = nullptr;
        e = cudaGetSymbolAddress((void**)&base, kvb_static_scratch);
        if (e != cudaSuccess) return (int)e;
        base_of_device[device] = base;
    }
    unsigned char* base = base_of_device[device];
    int* ticket_ptr = reinterpret_cast<int*>(base + (KVB_STATIC_SCRATCH_BYTES - KVB_STATIC_TICKET_BYTES));
    e = cudaMemsetAsync(ticket_ptr, 0, tickets * sizeof(int), stream);   // tickets start at zero, whatever the last call left
    if (e != cudaSuccess) return (int)e;
    return kvb_flash_decode(q, out, k_pages, v_pages, block_table, table_stride, items, n_items, seg_q_start, seg_q_len,
                            seg_kv_len, reinterpret_cast<float*>(base), ticket_ptr, Hq, Hkv, page_size, window, nsplit,
                            scale, stream);
}
