// Causal attention over cache pages for portions of prompts on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128; compiled per head size with -DKVB_HEAD_DIM).
//
// It computes what the reference's k_paged_attn computes (src/qwen_kernels.cu:146-185) and what this
// engine's mma.sync prefill kernel computes; on this GPU the warp-level mma.sync path tops out near a tenth
// of the tcgen05 rate, so long portions go through here.
//
// A piece of work is (unit, query head): a tile of 128 query positions of one segment, or a share of its key tiles; a
// thread of warps 0-3 owns one row.  The grid is as many blocks as the GPU holds at once, and a block takes pieces from
// a queue until none is left.
//   S = Q K^T   tcgen05.mma, M 128 x N 64 keys x K head size; Q and the key tile in 128-byte-swizzled shared
//               memory (K-major), brought by TMA - the key tile page by page through the block table;
//               S lands in tensor memory, 128 lanes x 64 columns.
//   softmax     each thread reads its row of S with tcgen05.ld, masks it (causal limit, window), keeps the running
//               maximum and sum in base 2 (the reference's recurrence, src/qwen_kernels.cu:159-176), and writes
//               P = 2^(s - m) as bfloat16 back into tensor memory (tcgen05.st), over the columns that held S.
//   O_t = P V   tcgen05.mma, M 128 x N head size x K 64 keys; P is the A operand, read from tensor memory, the value
//               tile as TMA left it - rows of keys, head size contiguous - is the B operand in MN-major form.
//               The thread adds its row of O_t (tcgen05.ld) into float32 registers, o = o * 2^(m_old - m_new) + O_t.
// S, P and O_t exist twice: while the threads run the softmax of tile i + 1, the tensor core multiplies P V of
// tile i and Q K^T of tile i + 2, and a thread adds O_t of tile i only after it has handed over P of tile i + 1 -
// so the softmax threads never wait for an MMA they have just asked for.
// Warp 4 brings the keys in and issues Q K^T, warp 5 brings the values in and issues P V, each through a ring of four
// stages.  What the two may cost is set by what the primitives cost on this GPU (measured on an idle SM; two to three
// times that beside the softmax warps): a wait on an mbarrier that has long completed 80 clocks when all lanes ask,
// 160 when one lane asks and tells the others; a shuffle 37, a vote 49; issuing one page's TMA copy 55; an MMA of this
// shape is accepted 48 clocks after the one before it (88 with two blocks on the SM), a commit 47.  One warp that did
// all of it - three waits, eight MMAs, four commits, eight copies a tile - needed longer for a tile than the softmax,
// and the block waited for it.  So each warp asks only the barriers it must (a stage is known to be free from barriers
// the warp has asked anyway: see AHEAD below), all lanes ask them, no barrier is committed that nobody needs, and a
// page that is not there is copied from before the pool's first row, which TMA fills with zeros, instead of being
// voted on and cleared by hand.
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
constexpr int SUB_BYTES = BQ * 128;                  // a [128 rows x 64 columns] bfloat16 sub-tile of Q, swizzled
constexpr int KV_SUB_BYTES = BKEYS * 128;            // a [64 keys x 64 columns] sub-tile (K, V)
constexpr int Q_BYTES = HALVES * SUB_BYTES, KV_BYTES = HALVES * KV_SUB_BYTES;
constexpr int STAGES = 4;                            // of keys, and of values: two rings, each filled on its own
static_assert(STAGES == 4, "the helper warps reuse a stage two tiles after its MMA without asking a barrier");
constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * KV_BYTES + 1024;
constexpr int TMEM_COLS = D == 64 ? 256 : 512;       // S: 2 x 64 columns, O_t: 2 x D columns
constexpr int THREADS = 192;                         // warps 0-3: softmax rows; warp 4: keys and Q K^T; warp 5: values and P V
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
    const int* units;          // [n_units, 8]: segment, first row of the tile, unit, units of the tile, tile id, first unit of the tile
    float* part_o;             // [units, Hq, D / 4, 128, 4]  unnormalised outputs of units that share a tile
    float* part_ml;            // [units, Hq, 128, 2]  their running maximum and sum
    int* tickets;              // [tiles, Hq], zero between launches
    int* queue;                // [2]: the next piece of work to hand out, and how many blocks have left; zero between launches
    int n_work;                // units * Hq pieces of work: (unit, head), the heads of a unit next to each other
    const int* seg_q_start;
    const int* seg_q_len;
    const int* seg_kv_len;
    int table_stride, Hq, Hkv, page_size, page_shift, window;
    float scale_log2;
    int* err;
};

struct Shared {
    uint64_t q_full, k_full[STAGES], v_full[STAGES], s_full[2], p_ready[2], o_full[2];
    uint32_t tmem_base;
    int failed;
    int work;                  // the piece of work the block is on
};

__global__ void __launch_bounds__(THREADS, D == 64 ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = base;
    unsigned char* k_s = q_s + Q_BYTES;                       // key stage s at k_s + s KV_BYTES
    unsigned char* v_s = k_s + STAGES * KV_BYTES;             // value stage s at v_s + s KV_BYTES
    __shared__ Shared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __shared__ int ticket_s;
    if (tid == 0) {
        mbar_init(&sh.q_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.k_full[s], 1); mbar_init(&sh.v_full[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.s_full[b], 1); mbar_init(&sh.p_ready[b], 128); mbar_init(&sh.o_full[b], 1); }
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
    const uint32_t tmem_s = sh.tmem_base, tmem_o = sh.tmem_base + 2 * BKEYS;   // S of tile g at + (g % 2) * 64, O_t at + (g % 2) * D

    // The block takes pieces of work from a queue until none is left: the grid is as many blocks as the GPU holds at once,
    // and a block that had a short piece takes another (a grid of one block per piece left the last pieces waiting for
    // places long after the first blocks had gone).  Buffers, stages and barrier phases go by g, the count of key tiles
    // the block has been through, so the pipeline's bookkeeping runs on from one piece to the next.
    int g0 = 0, units_done = 0, units_seen = 0;
    for (;;) {
    if (tid == 0) sh.work = atomicAdd(p.queue, 1);
    __syncthreads();
    const int work = sh.work;
    if (work >= p.n_work || sh.failed) break;
    const int unit = work / p.Hq, h = work - unit * p.Hq;
    const int* u = p.units + 8 * unit;
    const int seg = u[0], row0 = u[1], split = u[2], nsplit = u[3], tile_id = u[4], unit0 = u[5];
    const int hk = h / (p.Hq / p.Hkv);
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int first_pos = kv_len - q_len;
    const int tile_rows = min(BQ, q_len - row0);
    const int pos_first = first_pos + row0, pos_last = pos_first + tile_rows - 1;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    // The tile's key tiles are shared out among its units; a window may leave some units without any.
    const int tile_begin = key_lo / BKEYS, tile_end = pos_last / BKEYS + 1;
    const int per_split = (tile_end - tile_begin + nsplit - 1) / nsplit;
    const int n_valid = (tile_end - tile_begin + per_split - 1) / per_split;
    const int kt_begin = tile_begin + split * per_split, kt_end = min(tile_end, kt_begin + per_split);
    const int n = kt_end - kt_begin;

    // Everything up to here - barriers, tensor memory, the first piece and its record, which the host wrote at the start of
    // the step - has needed nothing of the kernel before (the rotation and append, which lets this one start early).
    if (units_seen++ == 0) { pdl_wait(); pdl_launch_dependents(); }
    if (split < n_valid) {       // else a window has left this unit without keys

    if (warp >= 4) {
        // ---- warp 4: keys and S = Q K^T; warp 5: values and O_t = P V.  Its first lanes copy a page each of a tile, its
        // first lane issues the MMAs; every lane waits on the barriers (a wait by one lane and a broadcast costs twice
        // as much). ----
        const bool keys = warp == 4;
        const int* table = p.block_table + (size_t)seg * p.table_stride;
        const int pages_per_tile = BKEYS >> p.page_shift;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        unsigned char* ring = keys ? k_s : v_s;
        uint64_t* full = keys ? sh.k_full : sh.v_full;
        bool ok = true;
        // Lane pg's page of tile kt_begin + j, looked up one tile before it is wanted.  Where the rows can see none of a
        // page's keys, or the table holds none, the copy is aimed before the pool's first row: the TMA unit fills what
        // lies outside the tensor with zeros (0 * NaN would poison the sums) and still counts the bytes.
        auto lookup = [&](int j) -> int {
            int page = -1;
            if (lane < pages_per_tile && j < n) {
                const int first_key = (kt_begin + j) * BKEYS + lane * p.page_size;
                if (first_key <= pos_last && first_key + p.page_size > key_lo) page = table[first_key >> p.page_shift];
            }
            return page;
        };
        // Tile kt_begin + j into stage j % STAGES; the caller has seen the MMA that read the stage's last tenant finish.
        auto load_tile = [&](int j, int my_page) {
            const int s = (g0 + j) % STAGES;
            unsigned char* dst = ring + (size_t)s * KV_BYTES;
            if (lane == 0) mbar_expect_tx(&full[s], KV_BYTES);
            __syncwarp();
            if (lane < pages_per_tile) {                                // lane pg copies page pg: the copies go out side by side
                const int row = my_page >= 0 ? (my_page * p.Hkv + hk) * p.page_size : -p.page_size;   // of the pool as [pages * heads * page, D]
#pragma unroll
                for (int hb = 0; hb < HALVES; ++hb)
                    tma_load_2d(dst + hb * KV_SUB_BYTES + lane * p.page_size * 128, map, hb * 64, row, &full[s]);
            }
        };
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
            if (keys) {
                asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
                mbar_expect_tx(&sh.q_full, Q_BYTES);
                for (int hb = 0; hb < HALVES; ++hb) tma_load_2d(q_s + hb * SUB_BYTES, &map_q, h * D + hb * 64, q_start + row0, &sh.q_full);
            }
        }
        // Tile i + AHEAD is asked for after the MMA of tile i has been issued, into the stage that tile i - 2 had.  No
        // barrier needs to be asked whether that stage is free: the keys' warp has just seen O_{i-2}, which was made from
        // P_{i-2} and so after S_{i-2}; the values' warp has just seen P_i handed over, and every thread that hands P_i
        // over has added O_{i-2} before.
        constexpr int AHEAD = STAGES - 2;
        int page_next = lookup(0);
        for (int j = 0; j < AHEAD && j < n; ++j) {
            const int page = page_next;
            page_next = lookup(j + 1);
            load_tile(j, page);
        }
        constexpr uint32_t idesc_s = instr_desc(BQ, BKEYS);
        constexpr uint32_t idesc_o = instr_desc(BQ, D) | (1u << 16);            // B (values) is MN-major
        if (keys) ok = mbar_wait(&sh.q_full, units_done & 1);
        for (int i = 0; i < n; ++i) {
            const int g = g0 + i, s = g % STAGES;
            if (keys) {
                // S_{g % 2} = Q K_i^T, once K_i is there and P of two tiles ago, which lies over S_{g % 2}, has been multiplied.
                ok = ok && mbar_wait(&sh.k_full[s], (g / STAGES) & 1);
                if (g >= 2) ok = ok && mbar_wait(&sh.o_full[g & 1], ((g - 2) >> 1) & 1);
            } else {
                // O_{g % 2} = P_i V_i, once the softmax threads have handed P_i over (O_{g % 2} is free then) and V_i is there.
                ok = ok && mbar_wait(&sh.p_ready[g & 1], (g >> 1) & 1);
                ok = ok && mbar_wait(&sh.v_full[s], (g / STAGES) & 1);
            }
            if (!ok) break;                                      // every lane asks the same barriers: they give up together, or nearly
            if (lane == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (keys) {
                    const uint32_t k_addr = smem_u32(k_s + (size_t)s * KV_BYTES);
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)               // 16 of the head size a step; 64 a sub-tile
                        umma(tmem_s + (g & 1) * BKEYS, smem_desc(smem_u32(q_s) + (k / 4) * SUB_BYTES) + 2 * (k % 4),
                             smem_desc(k_addr + (k / 4) * KV_SUB_BYTES) + 2 * (k % 4), idesc_s, k != 0 ? 1u : 0u);
                    umma_commit(&sh.s_full[g & 1]);
                } else {
                    const uint32_t v_addr = smem_u32(v_s + (size_t)s * KV_BYTES);
#pragma unroll
                    for (int k = 0; k < BKEYS / 16; ++k)           // 16 keys a step: 8 columns of P in tensor memory, 2048 bytes down V
                        umma_a_tmem(tmem_o + (g & 1) * D, tmem_s + (g & 1) * BKEYS + 8 * k,
                                    smem_desc_mn(v_addr + k * 2048, KV_SUB_BYTES), idesc_o, k != 0 ? 1u : 0u);
                    umma_commit(&sh.o_full[g & 1]);
                }
            }
            __syncwarp();
            if (i + AHEAD < n) {
                const int page = page_next;
                page_next = lookup(i + AHEAD + 1);
                load_tile(i + AHEAD, page);
            }
        }
        if (!ok && lane == 0) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; }
        __syncwarp();
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
        auto store_row = [&](const float* vals, float factor) {
            bf16* orow = p.out + ((size_t)(q_start + row0 + row) * p.Hq + h) * D;
#pragma unroll
            for (int d = 0; d < D; d += 8) {
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(vals[d + 2 * e] * factor, vals[d + 2 * e + 1] * factor);
                    w4[e] = *reinterpret_cast<uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(orow + d) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
        };
        float corr_prev = 1.f;                                  // the rescaling that belongs to the O_t not yet added
#ifdef KVB_TRACE
        long long c_wait_s = 0, c_soft = 0, c_wait_o = 0, c_add = 0, c_t, c_start = clock64();
#define TCLK(acc) { const long long now_ = clock64(); acc += now_ - c_t; c_t = now_; }
#define TCLK0() c_t = clock64();
#else
#define TCLK(acc)
#define TCLK0()
#endif
        // o = o * corr + O_t of tile i (from tensor memory).
        auto add_output = [&](int i, float corr) -> bool {   // i: the tile's count g
            TCLK0()
            if (!mbar_wait(&sh.o_full[i & 1], (i >> 1) & 1)) return false;
            TCLK(c_wait_o)
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {                      // two loads in flight: the scores' registers are free by now
                uint32_t r[64];
                tmem_ld32_nowait(tmem_o + (i & 1) * D + lane_base + c * 64, r);
                tmem_ld32_nowait(tmem_o + (i & 1) * D + lane_base + c * 64 + 32, r + 32);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 64; ++e) o[c * 64 + e] = fmaf(o[c * 64 + e], corr, __uint_as_float(r[e]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            TCLK(c_add)
            return true;
        };
        for (int i = 0; i < n; ++i) {
            const int g = g0 + i;
            TCLK0()
            ok = mbar_wait(&sh.s_full[g & 1], (g >> 1) & 1);
            if (!ok) break;
            TCLK(c_wait_s)
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int key0 = (kt_begin + i) * BKEYS;
            // Whether every row of this warp sees every key of the tile (then no element needs its mask).
            const bool open = pos >= 0 && key0 + BKEYS - 1 <= pos && (p.window <= 0 || key0 > pos - p.window);
            const bool warp_open = __all_sync(0xffffffffu, open);
            // The row of S, read once.
            uint32_t sv[BKEYS];
            tmem_ld32_nowait(tmem_s + (g & 1) * BKEYS + lane_base, sv);
            tmem_ld32_nowait(tmem_s + (g & 1) * BKEYS + lane_base + 32, sv + 32);
            tmem_ld_wait();
            if (!warp_open) {
#pragma unroll
                for (int e = 0; e < BKEYS; ++e) {
                    const int j = key0 + e;
                    const bool seen = j <= pos && (p.window <= 0 || j > pos - p.window);
                    if (!seen) sv[e] = __float_as_uint(NEG_INF);
                }
            }
            // The maximum over four chains of sixteen, not one of sixty-four: a maximum does not depend on the order.
            float mx4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
            for (int e = 0; e < BKEYS; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float base_m = m_new == NEG_INF ? 0.f : m_new;
            const float corr = ex2(m - base_m);
            m = m_new;
            l *= corr;
            // P = 2^(s * scale - m) as bfloat16 into tensor memory, over the first half of the columns that held this
            // tile's S (every score of the row is in registers by now): keys 2c and 2c + 1 of the row in column c, where
            // the product P V reads its A operand.  Shared memory carries neither P's stores nor the product's reads
            // of it.  A masked score is -inf and gives 0.
            float l4[4] = {0.f, 0.f, 0.f, 0.f};                 // four chains of additions; joined in one fixed order below
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t packed[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p0 = ex2(fmaf(__uint_as_float(sv[32 * half + 2 * c]), p.scale_log2, -base_m));
                    const float p1 = ex2(fmaf(__uint_as_float(sv[32 * half + 2 * c + 1]), p.scale_log2, -base_m));
                    l4[c & 3] += p0 + p1;
                    __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                    packed[c] = *reinterpret_cast<uint32_t*>(&v);
                }
                tmem_st16(tmem_s + (g & 1) * BKEYS + lane_base + 16 * half, packed);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tmem_st_wait();
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&sh.p_ready[g & 1]);
            TCLK(c_soft)
            // While the tensor core multiplies P_i V_i, add the O_t of the tile before.
            if (i >= 1) {
                ok = add_output(g - 1, corr_prev);
                if (!ok) break;
            }
            corr_prev = corr;
        }
        if (ok) ok = add_output(g0 + n - 1, corr_prev);
#ifdef KVB_TRACE
        if (tid == 0) {
            const int cta = work;
            if (cta < 8192) {
                long long* t = kvb_trace_buf + cta * 8;
                t[0] = n; t[1] = c_wait_s; t[2] = c_soft; t[3] = c_wait_o; t[4] = c_add; t[5] = clock64() - c_start;
                unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid)); t[6] = smid;
                t[7] = trace_now();
            }
        }
#endif
        if (!ok && lane == 0) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; }
        if (ok && n_valid == 1 && row < tile_rows) store_row(o, l > 0.f ? 1.f / l : 0.f);
        if (ok && n_valid > 1) {
            // Leave this unit's (m, l, o) for the block that merges the tile.
            // Layout [D / 4][128 rows] of float4, so that a warp's rows make one contiguous store.
            float4* po = reinterpret_cast<float4*>(p.part_o + ((size_t)(unit0 + split) * p.Hq + h) * BQ * D) + row;
#pragma unroll
            for (int d = 0; d < D; d += 4) po[(d / 4) * BQ] = make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]);
            *reinterpret_cast<float2*>(p.part_ml + (((size_t)(unit0 + split) * p.Hq + h) * BQ + row) * 2) = make_float2(m, l);
            __threadfence();
        }
        if (n_valid > 1) {
            asm volatile("bar.sync 1, 128;\n" ::: "memory");            // the four softmax warps
            if (tid == 0) ticket_s = atomicAdd(p.tickets + tile_id * p.Hq + h, 1);
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (ticket_s == n_valid - 1) {
                // The last unit of the tile to finish merges all of them, in unit order:
                // weight_s = 2^(m_s - M) / sum_s 2^(m_s - M) l_s, out = sum_s weight_s o_s.
                __threadfence();
                if (tid == 0) p.tickets[tile_id * p.Hq + h] = 0;
                if (ok && row < tile_rows) {
                    // Every unit, this one too, is read back from scratch: one order of additions whichever unit is last.
                    const float* ml0 = p.part_ml + (((size_t)unit0 * p.Hq + h) * BQ + row) * 2;
                    const float4* po0 = reinterpret_cast<const float4*>(p.part_o + ((size_t)unit0 * p.Hq + h) * BQ * D) + row;
                    const size_t ml_step = (size_t)p.Hq * BQ * 2, po_step = (size_t)p.Hq * BQ * D / 4;
                    float M = NEG_INF;
                    for (int s2 = 0; s2 < n_valid; ++s2) M = fmaxf(M, __ldcg(ml0 + s2 * ml_step));
                    const float base_m = M == NEG_INF ? 0.f : M;
                    float L = 0.f;
                    for (int s2 = 0; s2 < n_valid; ++s2) {
                        const float2 ml = __ldcg(reinterpret_cast<const float2*>(ml0 + s2 * ml_step));
                        L += ex2(ml.x - base_m) * ml.y;
                    }
                    const float inv = L > 0.f ? 1.f / L : 0.f;
                    float acc[D];
#pragma unroll
                    for (int d = 0; d < D; ++d) acc[d] = 0.f;
                    for (int s2 = 0; s2 < n_valid; ++s2) {
                        const float ws = ex2(__ldcg(ml0 + s2 * ml_step) - base_m) * inv;
                        const float4* po = po0 + s2 * po_step;
#pragma unroll
                        for (int d = 0; d < D; d += 4) {
                            const float4 v = __ldcg(po + (d / 4) * BQ);
                            acc[d] += ws * v.x; acc[d + 1] += ws * v.y; acc[d + 2] += ws * v.z; acc[d + 3] += ws * v.w;
                        }
                    }
                    store_row(acc, 1.f);
                }
            }
        }
    }

    g0 += n;
    ++units_done;
    }   // split < n_valid
    // Every MMA and copy of the piece has been waited for by someone; nobody goes on to the next piece (and to Q's place in
    // shared memory, and to sh.work) before all are here.
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    }   // pieces of work
    if (tid == 0) {
        // The last block to leave puts the queue back for the next launch.
        __threadfence();
        if (atomicAdd(p.queue + 1, 1) == (int)gridDim.x - 1) { p.queue[0] = 0; p.queue[1] = 0; }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && tid == 0) {      // give copies that may still be in flight a bounded chance to land
        mbar_wait(&sh.q_full, 0);
        for (int s = 0; s < STAGES; ++s) { mbar_wait(&sh.k_full[s], 0); mbar_wait(&sh.v_full[s], 0); }
    }
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(sh.tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace atc

KVB_API int kvb_attention_tc_head_dim() { return atc::D; }

KVB_API long long kvb_attention_tc_scratch_floats(int n_units, int Hq) {
    return (long long)n_units * Hq * atc::BQ * (atc::D + 2);
}

// q, out: [T, Hq * D] bfloat16; k_pages, v_pages: [num_pages, Hkv, page_size, D]; units: int32 [n_units, 8]
// (segment, first row of a tile of 128 rows, unit, units of the tile, tile id, first unit of the tile, 0, 0);
// scratch: kvb_attention_tc_scratch_floats floats; tickets: two ints (the work queue) and one per (tile, head), zero
// before the first launch (the kernel leaves them zero).  page_size a power of two, 8..64.
KVB_API int kvb_attention_tc(const void* q, void* out, const void* k_pages, const void* v_pages, int num_pages,
                             const int* block_table, int table_stride, const int* units, int n_units, float* scratch,
                             int* tickets, const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, int T,
                             int Hq, int Hkv, int page_size, int window, float scale, int* err, cudaStream_t stream) {
    using namespace atc;
    if (n_units <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq > 65535) return KVB_ERR_SHAPE;
    if (page_size < 8 || page_size > atc::BKEYS || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return KVB_ERR_ALIGN;
    CUtensorMap mq, mk, mv;
    int rc = make_bf16_map(&mq, q, T, Hq * D, (long long)Hq * D, BQ);
    if (rc != KVB_OK) return rc;
    const long long pool_rows = (long long)num_pages * Hkv * page_size;
    rc = make_bf16_map(&mk, k_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    rc = make_bf16_map(&mv, v_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    Params p;
    p.out = (bf16*)out; p.block_table = block_table; p.units = units; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.part_o = scratch; p.part_ml = scratch + (size_t)n_units * Hq * BQ * D;
    p.queue = tickets; p.tickets = tickets + 2; p.n_work = n_units * Hq;
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
    const int places = kvb_sm_count() * (D == 64 ? 2 : 1);       // blocks the GPU holds at once (shared memory, registers, tensor memory)
    dim3 grid(p.n_work < places ? p.n_work : places);
    kvb_launch(attention_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, stream, mq, mk, mv, p);
    return kvb_launch_status();
}
