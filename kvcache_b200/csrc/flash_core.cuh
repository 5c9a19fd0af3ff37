// Warp-level core of the bfloat16 attention kernels over cache pages: a warp owns 16 query
// rows, keys and values arrive in shared memory 64 keys at a time (cp.async, rows padded by
// 16 bytes so that ldmatrix is free of bank conflicts for every head size), scores and the
// weighted sum run on the tensor cores (mma.sync m16n8k16, float32 accumulators), and the
// softmax is the running (max, sum, acc) form of the reference
// (src/qwen_kernels.cu:159-176; split merge src/flash_decode.cu:82-101), in base 2.
//
// Compiled once per head size: KVB_HEAD_DIM is given on the command line (a multiple of 16,
// at most 128; larger heads use the generic kernel).
#pragma once
#include "common.cuh"

#ifndef KVB_HEAD_DIM
#error "compile with -DKVB_HEAD_DIM=<head size>"
#endif

namespace flash {

constexpr int D = KVB_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 128, "head sizes 16..128 in steps of 16");
constexpr int CHUNKS = D / 8;        // 16-byte chunks in a row
constexpr int STRIDE = D + 8;        // elements between rows in shared memory (one chunk of padding)
constexpr int KT = 64;               // keys in a tile
constexpr int KS = D / 16;           // k-steps of Q.K^T
constexpr int NT_O = D / 8;          // 8-wide column tiles of the output
constexpr int TILE_ELEMS = KT * STRIDE;
constexpr float NEG_INF = -INFINITY;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Where the keys of one (request, kv head) lie.
struct KVSource {
    const bf16* k_pages;
    const bf16* v_pages;
    const int* table;      // the request's row of the block table
    int hk, Hkv, page_size, page_shift;
};

// Copies keys/values [key0, key0 + KT) into a stage; keys >= key_end (or before key_lo) are zero-filled.
// Called by a block of 128 threads: two threads share a row and take alternate 16-byte chunks, so
// neighbours fetch one 32-byte sector together and each thread looks its page up once.
__device__ __forceinline__ void load_tile(bf16* ks, bf16* vs, const KVSource& src, int key0, int key_lo, int key_end) {
    const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int j = key0 + row;
    const bool valid = j >= key_lo && j < key_end;
    size_t off = 0;
    if (valid) {
        const int page = __ldg(src.table + (j >> src.page_shift));
        off = (((size_t)page * src.Hkv + src.hk) * src.page_size + (j & (src.page_size - 1))) * D;
    }
    const bf16* kg = src.k_pages + off;
    const bf16* vg = src.v_pages + off;
    bf16* kd = ks + row * STRIDE;
    bf16* vd = vs + row * STRIDE;
#pragma unroll
    for (int c = 0; c < CHUNKS / 2; ++c) {
        const int e = (2 * c + half) * 8;
        cp_async16(kd + e, kg + e, valid);
        cp_async16(vd + e, vg + e, valid);
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The 16 query rows of a warp.
struct WarpRows {
    uint32_t q[KS][4];     // A fragments of Q
    float o[NT_O][4];      // output accumulators: [.][0..1] row g, [.][2..3] row g + 8
    float m[2], l[2];      // running maximum (base-2 units) and this thread's share of the running sum
    int pos[2];            // absolute position of rows g and g + 8 (-1: the row does not exist)
};

__device__ __forceinline__ void rows_init(WarpRows& w) {
#pragma unroll
    for (int i = 0; i < NT_O; ++i) w.o[i][0] = w.o[i][1] = w.o[i][2] = w.o[i][3] = 0.f;
    w.m[0] = w.m[1] = NEG_INF;
    w.l[0] = w.l[1] = 0.f;
}

// Loads the Q fragments: `row_ptr(r)` gives the global address of row r's D elements, or nullptr.
template <typename RowPtr>
__device__ __forceinline__ void rows_load_q(WarpRows& w, RowPtr row_ptr) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bf16* r0 = row_ptr(g);
    const bf16* r1 = row_ptr(g + 8);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int d = ks * 16 + 2 * t;
        w.q[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + d) : 0u;
        w.q[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + d) : 0u;
        w.q[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + d + 8) : 0u;
        w.q[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + d + 8) : 0u;
    }
}

// Where element (row, col) of a key or value tile lies in shared memory; col is a multiple of 8 (ldmatrix
// takes 16 bytes of a row per lane).
struct PaddedTile {            // rows STRIDE elements apart (cp.async fills it)
    const bf16* base;
    __device__ __forceinline__ const bf16* at(int row, int col) const { return base + row * STRIDE + col; }
};
struct SwizzledTile {          // as TMA leaves it with the 128-byte swizzle: rows of 64 elements (128 bytes), whose 16-byte
    const unsigned char* base; // chunk c sits at chunk position c ^ (row % 8); the next 64 columns lie `half_bytes` further.
    int half_bytes;            // `base` is 1024-byte aligned.
    __device__ __forceinline__ const bf16* at(int row, int col) const {
        return reinterpret_cast<const bf16*>(base + (col >> 6) * half_bytes + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4));
    }
};

// NK keys [key0, key0 + NK) whose rows start at row 0 of `kt` / `vt`: scores, masking, running
// softmax, weighted sum.  NK is a multiple of 16 (a whole tile, or a part of one).
// A key j is seen by a row at position p iff key_lo(p) <= j <= p, key_lo(p) = max(0, p - window + 1).
// MASKED = false: the caller knows that every row sees every key of the range.
template <int NK, bool MASKED, class Tile>
__device__ __forceinline__ void rows_tile(WarpRows& w, const Tile& kt, const Tile& vt, int key0, int window,
                                          float scale_log2) {
    const int lane = threadIdx.x & 31, t = lane & 3;
    float s[NK / 8][4];
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
        const int mi = lane >> 3, key_off = (mi >> 1) * 8 + (lane & 7), d_off = (mi & 1) * 8;
#pragma unroll
        for (int k = 0; k < KS; ++k) {
#pragma unroll
            for (int n2 = 0; n2 < NK / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, kt.at(n2 * 16 + key_off, k * 16 + d_off));
                mma_bf16(s[2 * n2], w.q[k], b0, b1);
                mma_bf16(s[2 * n2 + 1], w.q[k], b2, b3);
            }
        }
    }
    // Row maxima of the raw scores (masked ones count as -inf); scores stay unscaled until the exponent.
    float mx[2] = {NEG_INF, NEG_INF};
#pragma unroll
    for (int n = 0; n < NK / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (MASKED) {
                const int j = key0 + n * 8 + 2 * t + (e & 1);
                const int p = w.pos[e >> 1];
                const bool seen = j <= p && (window <= 0 || j > p - window);
                if (!seen) s[n][e] = NEG_INF;
            }
            mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
        }
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(w.m[r], mx[r] * scale_log2);      // scale_log2 > 0: the maximum commutes with it
        base[r] = m_new == NEG_INF ? 0.f : m_new;
        corr[r] = ex2(w.m[r] - base[r]);
        w.m[r] = m_new;
        w.l[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < NK / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = ex2(fmaf(s[n][e], scale_log2, -base[e >> 1]));
            s[n][e] = p;
            w.l[e >> 1] += p;
        }
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // the maxima seldom move once a few tiles are in
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            w.o[i][0] *= corr[0]; w.o[i][1] *= corr[0];
            w.o[i][2] *= corr[1]; w.o[i][3] *= corr[1];
        }
    }
    {
        const int mi = lane >> 3, key_off = (mi & 1) * 8 + (lane & 7), d_off = (mi >> 1) * 8;
#pragma unroll
        for (int kk = 0; kk < NK / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < NT_O / 2; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, vt.at(kk * 16 + key_off, n2 * 16 + d_off));
                mma_bf16(w.o[2 * n2], pa, b0, b1);
                mma_bf16(w.o[2 * n2 + 1], pa, b2, b3);
            }
        }
    }
}

// NK keys from key0 on: masked only if a row may miss one of them.  `pos_min` / `pos_max`: smallest and
// largest position among the warp's existing rows.
template <int NK, class Tile>
__device__ __forceinline__ void rows_tile_auto_in(WarpRows& w, const Tile& kt, const Tile& vt, int key0, int window,
                                               float scale_log2, int pos_min, int pos_max, bool all_rows_exist) {
    const bool open = all_rows_exist && key0 + NK - 1 <= pos_min && (window <= 0 || key0 > pos_max - window);
    if (open) rows_tile<NK, false>(w, kt, vt, key0, window, scale_log2);
    else rows_tile<NK, true>(w, kt, vt, key0, window, scale_log2);
}
template <int NK>
__device__ __forceinline__ void rows_tile_auto(WarpRows& w, const bf16* ks, const bf16* vs, int key0, int window,
                                               float scale_log2, int pos_min, int pos_max, bool all_rows_exist) {
    rows_tile_auto_in<NK>(w, PaddedTile{ks}, PaddedTile{vs}, key0, window, scale_log2, pos_min, pos_max, all_rows_exist);
}

// Sums each row's l over the four threads that share it.
__device__ __forceinline__ void rows_finish_sum(WarpRows& w) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        w.l[r] += __shfl_xor_sync(0xffffffffu, w.l[r], 1);
        w.l[r] += __shfl_xor_sync(0xffffffffu, w.l[r], 2);
    }
}

// Writes normalised rows: `row_ptr(r)` gives the output address of row r or nullptr.
template <typename RowPtr>
__device__ __forceinline__ void rows_store(const WarpRows& w, RowPtr row_ptr) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        bf16* out = row_ptr(g + 8 * r);
        if (!out) continue;
        const float inv = w.l[r] > 0.f ? 1.f / w.l[r] : 0.f;
#pragma unroll
        for (int i = 0; i < NT_O; ++i)
            *reinterpret_cast<uint32_t*>(out + i * 8 + 2 * t) = pack_bf16(w.o[i][2 * r] * inv, w.o[i][2 * r + 1] * inv);
    }
}

}  // namespace flash
