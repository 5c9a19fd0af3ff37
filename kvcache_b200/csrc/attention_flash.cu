// bfloat16 attention over cache pages on the tensor cores: a kernel for segments that bring
// few rows (decode: split over the keys, all query heads of a kv head in one warp) and a
// kernel for portions of prompts (64 query positions of one head per block).
//
// What they replace in the reference: k_batched_paged_decode_attn and k_paged_attn
// (src/qwen_kernels.cu:293-335, :146-185; one block of D threads per (query, head), serial
// over the keys with a tree reduction per key), with the split over the keys and its merge
// taken from the toy flash-decode kernel (src/flash_decode.cu:18-101).
#include "flash_core.cuh"

using namespace flash;

#define DECODE_STAGES (KVB_HEAD_DIM <= 64 ? 3 : 2)
#define PREFILL_STAGES 2

// ---------------------------------------------------------------------------------------------
// Decode: one warp per (item, kv head, split).  An item is a segment whose rows * group <= 16:
// row r of the warp is query (r / G) of the segment, head hk * G + r % G, so keys and values
// are read once for all heads that share them.  Each split scans a range of key tiles and
// leaves (m, l, acc) in scratch; the last split to finish (a ticket counter per (item, kv head))
// merges them in split order and resets the counter.
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
};

__global__ void __launch_bounds__(32) flash_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    const int split = blockIdx.x, hk = blockIdx.y, item = blockIdx.z;
    const int seg = p.items ? p.items[item] : item;
    const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
    const int G = p.Hq / p.Hkv;
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int rows = q_len * G;
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
        if (s < n) load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (my_begin + s) * KT, key_lo, kv_len, lane, 32);
        cp_async_commit();
    }
    for (int i = 0; i < n; ++i) {
        const int ahead = i + STAGES - 1;
        if (ahead < n) {
            const int s = ahead % STAGES;
            load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (my_begin + ahead) * KT, key_lo, kv_len, lane, 32);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const int s = i % STAGES;
        rows_tile(w, smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, (my_begin + i) * KT, p.window, p.scale_log2);
        __syncwarp();
    }
    rows_finish_sum(w);

    auto out_row = [&](int r) -> bf16* {
        return r < rows ? p.out + ((size_t)(q_start + r / G) * p.Hq + hk * G + r % G) * D : nullptr;
    };
    if (n_valid == 1) {
        rows_store(w, out_row);
        return;
    }
    // Leave this split's partial result, then take a ticket.
    const size_t slot = ((size_t)item * p.Hkv + hk) * p.nsplit;
    float* po = p.part_o + (slot + split) * 16 * D;
    float* pml = p.part_ml + (slot + split) * 16 * 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int i = 0; i < NT_O; ++i)
            *reinterpret_cast<float2*>(po + row * D + i * 8 + 2 * t) = make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
        if (t == 0) { pml[row * 2] = w.m[r]; pml[row * 2 + 1] = w.l[r]; }
    }
    __threadfence();
    __syncwarp();
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(p.tickets + item * p.Hkv + hk, 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != n_valid - 1) return;
    __threadfence();
    if (lane == 0) p.tickets[item * p.Hkv + hk] = 0;
    // Merge: lane s holds split s (nsplit <= 32).  M = max m_s; weight_s = 2^(m_s - M) / sum_s 2^(m_s - M) l_s;
    // out = sum_s weight_s acc_s, added in split order.
    for (int row = 0; row < rows; ++row) {
        float ms = NEG_INF, ls = 0.f;
        if (lane < n_valid) {
            const float* ml = p.part_ml + ((slot + lane) * 16 + row) * 2;
            ms = __ldcg(ml);
            ls = __ldcg(ml + 1);
        }
        const float M = warp_max(ms);
        const float e = exp2f(ms - (M == NEG_INF ? 0.f : M));
        const float L = warp_sum(e * ls);
        const float weight = L > 0.f ? e / L : 0.f;
        bf16* o = out_row(row);
        for (int d0 = 0; d0 < D; d0 += 32) {
            const int d = d0 + lane;
            float acc = 0.f;
            for (int s = 0; s < n_valid; ++s) {
                const float ws = __shfl_sync(0xffffffffu, weight, s);
                if (d < D) acc += ws * __ldcg(p.part_o + ((slot + s) * 16 + row) * D + d);
            }
            if (d < D) o[d] = __float2bfloat16_rn(acc);
        }
    }
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
    if (nsplit < 1 || nsplit > 32 || n_items > 65535 || Hkv > 65535) return KVB_ERR_LIMIT;
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
    const size_t smem = (size_t)DECODE_STAGES * 2 * TILE_ELEMS * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nsplit, Hkv, n_items);
    flash_decode_kernel<<<grid, 32, smem, stream>>>(p);
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Prefill: one block of four warps per (tile, query head); a tile is 64 consecutive query
// positions of one segment (16 per warp).  Key tiles run from the first key the tile's first
// row sees to the last row's own position; a warp skips key tiles that none of its rows see.
// ---------------------------------------------------------------------------------------------
struct PrefillParams {
    const bf16* q;
    bf16* out;
    const bf16* k_pages;
    const bf16* v_pages;
    const int* block_table;
    const int* tiles;          // [n_tiles, 2]: segment, first row of the tile within the segment
    const int* seg_q_start;
    const int* seg_q_len;
    const int* seg_kv_len;
    int table_stride, Hq, Hkv, page_size, page_shift, window;
    float scale_log2;
};

__global__ void __launch_bounds__(128) flash_prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    const int tile = blockIdx.x, h = blockIdx.y;
    const int seg = p.tiles[2 * tile], row0 = p.tiles[2 * tile + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
    const int hk = h / (p.Hq / p.Hkv);
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int first_pos = kv_len - q_len;                    // position of the segment's first row
    const int tile_rows = min(64, q_len - row0);
    const int pos_first = first_pos + row0, pos_last = first_pos + row0 + tile_rows - 1;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int kt_begin = key_lo / KT, kt_end = pos_last / KT + 1;
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
        if (s < n) load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (kt_begin + s) * KT, key_lo, pos_last + 1, threadIdx.x, 128);
        cp_async_commit();
    }
    for (int i = 0; i < n; ++i) {
        const int ahead = i + STAGES - 1;
        if (ahead < n) {
            const int s = ahead % STAGES;
            load_tile(smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, src, (kt_begin + ahead) * KT, key_lo, pos_last + 1, threadIdx.x, 128);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const int s = i % STAGES;
        const int key0 = (kt_begin + i) * KT;
        if (warp_rows > 0 && key0 <= warp_pos_last && key0 + KT > warp_key_lo)
            rows_tile(w, smem + (2 * s) * TILE_ELEMS, smem + (2 * s + 1) * TILE_ELEMS, key0, p.window, p.scale_log2);
        __syncthreads();
    }
    rows_finish_sum(w);
    auto out_row = [&](int r) -> bf16* {
        return wrow0 + r < q_len ? p.out + ((size_t)(q_start + wrow0 + r) * p.Hq + h) * D : nullptr;
    };
    rows_store(w, out_row);
}

KVB_API int kvb_flash_prefill(const void* q, void* out, const void* k_pages, const void* v_pages,
                              const int* block_table, int table_stride, const int* tiles, int n_tiles,
                              const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, int Hq, int Hkv,
                              int page_size, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (Hq > 65535) return KVB_ERR_LIMIT;
    PrefillParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.tiles = tiles; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len; p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = (size_t)PREFILL_STAGES * 2 * TILE_ELEMS * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, Hq);
    flash_prefill_kernel<<<grid, 128, smem, stream>>>(p);
    return kvb_launch_status();
}
