// Attention over the paged cache for prompt portions on the 5th-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory, TMA page loads), bfloat16, head size 64.
//
// The same work items as attention_mma.cu's wide shape: a tile of 128 query rows of one sequence
// and one kv head (rows are (token, query head of the group)) with a range of key positions.
// A block of 128 threads owns the tile: thread i owns row i, which is lane i of tensor memory.
// For every tile of 128 keys:
//   1. thread 0 waits for the K and V pages of the tile (one TMA box per page, 128-byte swizzle,
//      straight from the page pool through the block table) and issues s = q k^T: four
//      tcgen05.mma (M 128, N 128, K 16), accumulator s in tensor memory;
//   2. every thread reads its row of s (tcgen05.ld), masks (causal, window, range), keeps the
//      running maximum and sum in float32, and writes p = exp2(...) as bfloat16 into shared
//      memory in the operand layout (its row of two 64-key swizzled sub-tiles);
//   3. thread 0 issues o_tile = p v: eight tcgen05.mma (M 128, N 64, K 16) with v as the
//      "MN-major" operand, i.e. exactly as the cache stores it ([key][feature]);
//   4. every thread reads its row of o_tile and adds it to its float32 output row, scaled by the
//      change of the running maximum.
// While a tile is worked on, the pages of the next one are in flight (two stages).  Two blocks
// fit an SM (112 KB of shared memory, 256 of 512 tensor-memory columns each), so the softmax of
// one overlaps the matrix products of the other.
//
// Formulas as in src/layers/attention.py:35-71 (scale after the product, causal mask, float32
// softmax), grouped-query heads share the kv head's tiles.  Split key ranges write partial
// results in the layout `de_attn_combine` merges.
//
// Every mbarrier wait is bounded (status 3, the block then runs to its end and frees its tensor
// memory); no cluster launch, no multicast.

#include <cuda.h>

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int D = 64;                  // head size: 128 bytes of bfloat16 = one swizzle row
constexpr int ROWS = 128;              // query rows of a tile = lanes of tensor memory
constexpr int KT = 128;                // keys per tile
constexpr int THREADS = 128;
constexpr int TILE_BYTES = 128 * 128;  // 128 rows of 128 bytes
constexpr int TMEM_COLS = 256;         // s: 0..127, o_tile: 128..191
constexpr unsigned SPIN_LIMIT = 20u * 1000u * 1000u;
constexpr int PAGE_CACHE = 192;        // block-table entries kept in shared memory
constexpr int SMEM_BYTES = 7 * TILE_BYTES + 48 + PAGE_CACHE * 4;
#ifndef V_DESC_SWAP
#define V_DESC_SWAP 0
#endif

struct WorkItem {
    int seq, row0, kv_begin, kv_end, partial, pad0, pad1, pad2;
};

// ---------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* status) {
    const unsigned addr = smem_u32(bar);
    for (unsigned spins = 0; spins < SPIN_LIMIT; ++spins) {
        unsigned done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    atomicExch(status, 3);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, void* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(void* smem_result, unsigned columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned d_tmem, unsigned long long a_desc,
                                          unsigned long long b_desc, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((unsigned)accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_loads() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_load_32cols(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem),
                 "r"(bytes));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// K-major operand tile of rows x 64 bfloat16, 128-byte swizzle: groups of 8 rows are 1024 bytes
// apart (stride byte offset); see gemm_tcgen05.cu for the bit fields.
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand: the tile is stored [k][64 contiguous n] (v as the cache holds it: [key][feature]),
// 128-byte swizzle; groups of 8 k are 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
#if V_DESC_SWAP
    d |= (unsigned long long)(1024 >> 4) << 16;
    d |= (unsigned long long)1 << 32;
#else
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
#endif
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands, a K-major, b K-major or
// MN-major (bit 16), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr unsigned instr_desc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS)
attn_tcgen05_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                    int out_stride, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                    int table_stride, int num_pages, const int* __restrict__ seq_slot,
                    const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                    const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items,
                    float* __restrict__ partial_acc, float* __restrict__ partial_ml, int heads,
                    int kv_heads, int page, float scale, int window, int* status) {
    // All shared memory is dynamic and starts at the block's window (1024-byte aligned, which the
    // swizzled tiles need; checked below): seven tiles, then barriers, the tensor-memory address
    // and the block-table entries of this item's key range.  Two blocks fit an SM.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* q_s = smem_raw;                               // 16 KB
    unsigned char* k_s = q_s + TILE_BYTES;                       // 2 x 16 KB
    unsigned char* v_s = k_s + 2 * TILE_BYTES;                   // 2 x 16 KB
    unsigned char* p_s = v_s + 2 * TILE_BYTES;                   // 2 sub-tiles of 128 rows x 64 keys
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + 7 * TILE_BYTES);
    unsigned long long* kv_full = bars;                          // [2]
    unsigned long long& s_done = bars[2];
    unsigned long long& o_done = bars[3];
    unsigned& tmem_slot = *reinterpret_cast<unsigned*>(bars + 4);
    int* page_ids = reinterpret_cast<int*>(bars + 6);            // [PAGE_CACHE]

    const WorkItem it = items[blockIdx.x];
    if (it.kv_begin >= it.kv_end || (smem_u32(smem_raw) & 1023u) != 0) {   // padding item
        if ((smem_u32(smem_raw) & 1023u) != 0 && threadIdx.x == 0) atomicExch(status, 4);
        pdl_wait();
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;

    if (tid == 0) {
        mbar_init(&kv_full[0], 1);
        mbar_init(&kv_full[1], 1);
        mbar_init(&s_done, 1);
        mbar_init(&o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
    // stale shared memory must be finite: p = 0 times a NaN bit pattern would poison the product
    for (int i = tid; i < 4 * TILE_BYTES / 16; i += THREADS)
        reinterpret_cast<uint4*>(k_s)[i] = make_uint4(0u, 0u, 0u, 0u);

    // this thread's row
    const int r = it.row0 + tid;
    const bool live = r < rows_total;
    const int tok = live ? r / g : 0;
    const int hq = hk * g + (live ? r % g : 0);
    const int pos = live ? pos0 + tok : -1;

    // key range of the tile and of this row
    const int last_row = min(it.row0 + ROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    int k_lo_true = it.kv_begin;
    if (window > 0) k_lo_true = max(k_lo_true, min_pos - window + 1);
    const int k_lo = (k_lo_true / KT) * KT;
    int lo = it.kv_begin;
    if (window > 0) lo = max(lo, pos - window + 1);
    const int hi = min(it.kv_end, pos + 1);                      // dead row: nothing visible
    const int n_tiles = (k_hi - k_lo + KT - 1) / KT;

    // the block-table entries of the range, once, so that the loads below do not wait on them
    const int first_page = k_lo / page;
    const int range_pages = (k_hi + page - 1) / page - first_page;
    for (int i = tid; i < min(range_pages, PAGE_CACHE); i += THREADS)
        page_ids[i] = block_table[(size_t)slot * table_stride + first_page + i];

    pdl_wait();            // q, and the keys and values of this step's tokens, are just written

    // q row into shared memory, operand layout (chunk index xor row % 8)
    {
        const __nv_bfloat16* src = q + (size_t)(tok0 + tok) * q_stride + hq * D;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            cp_async16(q_s + tid * 128 + ((c ^ (tid & 7)) << 4), src + c * 8, live);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> tensor core
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem = tmem_slot;
    const unsigned tmem_s = tmem, tmem_o = tmem + 128;

    // pages of one tile: a TMA box per page that holds keys of the range; the lanes of warp 0 take
    // the pages in turn, lane 0 announces the bytes first
    const int pages_per_tile = KT / page;
    const unsigned page_bytes = (unsigned)page * 128u;
    auto page_of = [&](int index) {
        return index < PAGE_CACHE ? page_ids[index]
                                  : block_table[(size_t)slot * table_stride + first_page + index];
    };
    auto load_tile = [&](int tile, int stage) {                  // all lanes of warp 0
        const int kt = k_lo + tile * KT;
        unsigned mine = 0;
        for (int p = lane; p < pages_per_tile; p += 32) {
            const int first = kt + p * page;
            if (first + page <= k_lo_true || first >= k_hi) continue;
            const int id = page_of(first / page - first_page);
            if (id >= 0 && id < num_pages) mine += 2 * page_bytes;
        }
        unsigned bytes = mine;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
        if (lane == 0) mbar_expect_tx(&kv_full[stage], bytes);
        __syncwarp();
        for (int p = lane; p < pages_per_tile; p += 32) {
            const int first = kt + p * page;
            if (first + page <= k_lo_true || first >= k_hi) continue;
            const int id = page_of(first / page - first_page);
            if (id < 0 || id >= num_pages) continue;
            const int y = (id * kv_heads + hk) * page;
            tma_load_2d(k_s + stage * TILE_BYTES + p * page_bytes, &map_k, &kv_full[stage], 0, y);
            tma_load_2d(v_s + stage * TILE_BYTES + p * page_bytes, &map_v, &kv_full[stage], 0, y);
        }
    };

    float o_row[D];
#pragma unroll
    for (int j = 0; j < D; ++j) o_row[j] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    const float sl = scale * 1.4426950408889634f;
    constexpr unsigned idesc_s = instr_desc(128, 128, false);
    constexpr unsigned idesc_o = instr_desc(128, 64, true);
    bool ok = true;

    if (warp == 0) load_tile(0, 0);
    for (int tile = 0; tile < n_tiles && ok; ++tile) {
        const int stage = tile & 1;
        const int kt = k_lo + tile * KT;
        // the other stage was read by the products of tile - 1, which are complete (o_done)
        if (warp == 0 && tile + 1 < n_tiles) load_tile(tile + 1, stage ^ 1);
        if (tid == 0) {
            ok = mbar_wait(&kv_full[stage], (tile >> 1) & 1, status);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned long long a = desc_k_major(q_s);
                const unsigned long long b = desc_k_major(k_s + stage * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) umma_bf16(tmem_s, a + 2 * k, b + 2 * k, idesc_s, k > 0);
            }
            umma_commit(&s_done);
        }
        // ---- softmax of this thread's row
        ok = mbar_wait(&s_done, tile & 1, status);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        float corr = 1.0f;
        if (ok) {
            const unsigned lane_addr = tmem_s + ((unsigned)(warp * 32) << 16);
            unsigned sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_load_32cols(lane_addr + 32 * c, sv[c]);
            tmem_wait_loads();
            float m_new = m_run;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = kt + 32 * c + i;
                    float s = __uint_as_float(sv[c][i]);
                    if (key < lo || key >= hi) s = -INFINITY;
                    sv[c][i] = __float_as_uint(s);
                    m_new = fmaxf(m_new, s);
                }
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            corr = fast_exp2((m_run - m_use) * sl);
            m_run = m_new;
            float l_add = 0.0f;
            // p as bfloat16 into the operand layout: row tid of sub-tile (key / 64), 16-byte chunk
            // ((key % 64) / 8) xor (tid % 8)
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float p[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        p[j] = fast_exp2((__uint_as_float(sv[c][i + j]) - m_use) * sl);
                        l_add += p[j];
                    }
                    uint4 u;
                    u.x = pack2(p[0], p[1]); u.y = pack2(p[2], p[3]);
                    u.z = pack2(p[4], p[5]); u.w = pack2(p[6], p[7]);
                    const int key_in_tile = 32 * c + i;
                    const int sub = key_in_tile >> 6, chunk = (key_in_tile & 63) >> 3;
                    *reinterpret_cast<uint4*>(p_s + sub * TILE_BYTES + tid * 128 +
                                              ((chunk ^ (tid & 7)) << 4)) = u;
                }
            l_run = l_run * corr + l_add;
        }
        // Pages come whole: rows of v beyond the range (the rest of the last page, or keys before a
        // window) may hold anything, and 0 * NaN is NaN in the product.  Row tid of the stage is key
        // kt + tid: zero it when it lies outside the tile's range.
        if (ok && (kt + tid >= k_hi || kt + tid < k_lo_true)) {
            if (tid != 0) mbar_wait(&kv_full[stage], (tile >> 1) & 1, status);   // the pages have landed
            uint4* vrow = reinterpret_cast<uint4*>(v_s + stage * TILE_BYTES + tid * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        // ---- o_tile = p v
        if (tid == 0) {
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned long long b = desc_mn_major(v_s + stage * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < KT / 16; ++k) {
                    // 16 keys of p are 32 bytes inside a sub-tile row; 16 keys of v are 2 groups of
                    // 8 rows = 2048 bytes
                    const unsigned long long a = desc_k_major(p_s + (k >> 2) * TILE_BYTES) + 2 * (k & 3);
                    umma_bf16(tmem_o, a, b + (unsigned long long)(k * 2048 >> 4), idesc_o, k > 0);
                }
            }
            umma_commit(&o_done);
        }
        const bool got = mbar_wait(&o_done, tile & 1, status);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        ok = ok && got;
        if (ok) {
            const unsigned lane_addr = tmem_o + ((unsigned)(warp * 32) << 16);
            unsigned ov[2][32];
            tmem_load_32cols(lane_addr, ov[0]);
            tmem_load_32cols(lane_addr + 32, ov[1]);
            tmem_wait_loads();
#pragma unroll
            for (int j = 0; j < D; ++j)
                o_row[j] = o_row[j] * corr + __uint_as_float(ov[j >> 5][j & 31]);
        }
        // the block's votes differ only after a failed wait; leave the loop together (this is also
        // the barrier between this tile's reads of tensor memory and the next tile's products)
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        ok = __syncthreads_and(ok);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    }
    pdl_trigger();

    if (ok && live) {
        if (it.partial < 0) {
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            __nv_bfloat16* o = out + (size_t)(tok0 + tok) * out_stride + hq * D;
#pragma unroll
            for (int j = 0; j < D; j += 8) {
                uint4 u;
                u.x = pack2(o_row[j] * inv, o_row[j + 1] * inv);
                u.y = pack2(o_row[j + 2] * inv, o_row[j + 3] * inv);
                u.z = pack2(o_row[j + 4] * inv, o_row[j + 5] * inv);
                u.w = pack2(o_row[j + 6] * inv, o_row[j + 7] * inv);
                *reinterpret_cast<uint4*>(o + j) = u;
            }
        } else {
            const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + tid;
            float* pa = partial_acc + idx * D;
#pragma unroll
            for (int j = 0; j < D; j += 4)
                *reinterpret_cast<float4*>(pa + j) =
                    make_float4(o_row[j], o_row[j + 1], o_row[j + 2], o_row[j + 3]);
            partial_ml[idx * 2] = m_run * scale;                  // natural-log domain, as merged
            partial_ml[idx * 2 + 1] = l_run;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) ==
                cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

// the page pool of one layer as a matrix [pages * kv_heads * page rows, 64], boxes of one page
int make_page_map(CUtensorMap* map, const void* pages, long long rows, int page) {
    EncodeTiled encode = encode_fn();
    if (encode == nullptr) return -20;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {(cuuint32_t)D, (cuuint32_t)page};
    cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages),
                              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -21;
}

}  // namespace

DE_EXPORT int de_attn_tcgen05_rows() { return ROWS; }
DE_EXPORT int de_attn_tcgen05_head_dim() { return D; }

// Arguments as de_attn_mma (wide shape); `status` receives 3 if a wait inside the kernel ran out.
DE_EXPORT int de_attn_tcgen05(const void* q, int q_stride, void* out, int out_stride,
                              const void* k_pages, const void* v_pages, const int* block_table,
                              int table_stride, int num_pages, const int* seq_slot,
                              const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                              const int* items, int num_items, float* partial_acc,
                              float* partial_ml, int heads, int kv_heads, int head_dim, int page,
                              float scale, int window, int* status, void* stream) {
    if (num_items <= 0) return 0;
    if (head_dim != D || heads % kv_heads != 0) return -2;
    if (page <= 0 || KT % page != 0 || q_stride % 8 != 0 || out_stride % 8 != 0 ||
        ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_pages & 15) ||
        ((uintptr_t)v_pages & 15))
        return -3;
    CUtensorMap map_k, map_v;
    const long long rows = (long long)num_pages * kv_heads * page;
    int code = make_page_map(&map_k, k_pages, rows, page);
    if (code) return code;
    code = make_page_map(&map_v, v_pages, rows, page);
    if (code) return code;
    const size_t smem = SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(attn_tcgen05_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(num_items, kv_heads);
    return de_launch(attn_tcgen05_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream,
                     (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, map_k, map_v,
                     block_table, table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0,
                     (const WorkItem*)items, partial_acc, partial_ml, heads, kv_heads, page, scale,
                     window, status);
}
