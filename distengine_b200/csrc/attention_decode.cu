// Attention of decoded tokens in one launch per layer: every sequence of the step brings one token.
// bfloat16 on the tensor cores (mma.sync m16n8k16, as attention_mma.cu's narrow shape: a tile of 16
// rows, the rows being the query heads of one kv head's group, the 4 warps split the 64 keys of a
// key tile), float32 softmax.  Compiled once per head size (-DHEAD_DIM=d).
//
// What is folded in, so that a layer's attention is one kernel instead of four:
//   * rotation of q and of the token's own key (src/layers/rotary_embedding.py:45-54) and the store
//     of that key and value into the pages (src/distengine/paged_kv_cache.py:165-167).  A block
//     rotates its own query rows; the block whose key range holds the token's position rotates the
//     key, stores key and value (the block of the group's first rows only) and uses them from
//     shared memory, so nothing that this launch writes is read from the cache.  The qkv buffer is
//     left as the product wrote it.
//   * the merge of a split key range.  The chunks of a range are the blocks of one thread-block
//     cluster.  Every block owns a slice of the output's columns.  When all blocks of the cluster
//     are through their key tiles (first cluster barrier), every warp stores its unnormalised
//     result (accumulator, maximum, sum) straight from its registers into the owners' shared
//     memory (distributed shared memory, in the space the key tiles no longer need); after the
//     second barrier each owner merges its slice from its own shared memory and writes it out:
//     no block-level merge first, no remote loads, no trip through global memory.
//     Ranges longer than a cluster's reach take several clusters; each writes a partial result,
//     and the block that finishes last (a counter per tile and kv head, left at zero again)
//     merges them in the arithmetic of `de_attn_combine`.  No block spins on another: the cluster
//     barrier is the hardware's, and every block of a cluster reaches both barriers on every path.
//   * the cache rows of earlier tokens are requested before the kernel waits for the kernel before
//     it (programmatic dependent launch).  They were written by earlier steps: between their
//     writer and this launch lies at least one kernel that waited for its predecessor before it
//     let its successor start (this kernel itself does, in the layer before), so the writer has
//     completed.  That does not hold for a run that reads another run's cache (write_kv == 0):
//     the key of this step's own token was stored there by a kernel of this same step, possibly
//     with only early-triggering products in between, and is sure to be visible only after the
//     wait; such a run requests its tiles after the wait.
//
// Items (attention_plan): every tile has `cap` consecutive items (its chunks in ascending order,
// padded with empty ones), `cap` a multiple of the cluster size; block (g, hk, rank) of the grid
// takes item g * cluster + rank and kv head hk.  In place of the partial slots, which this kernel
// derives itself, an item carries the token's position and its sequence's slot.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

#include <cooperative_groups.h>

#include "attention_mma_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int WN = 4;                  // warps; they split the keys of a tile
constexpr int ROWS = 16;
constexpr int NK = KT / WN;
constexpr int NT = NK / 8;
constexpr int DT = D / 8;
constexpr int CHUNKS = D / 8;          // 16-byte pieces of a key's row
constexpr int MAX_CLUSTER = 8;
#ifndef DECODE_STAGES
#define DECODE_STAGES 2
#endif
constexpr int STAGES = DECODE_STAGES;  // key tiles in flight or in use

// shared memory, in bytes from the start (all offsets multiples of 16)
constexpr int OFF_K = 0;                                         // [STAGES][KT][LDS] bf16
constexpr int OFF_V = OFF_K + STAGES * KT * LDS * 2;             // [STAGES][KT][LDS] bf16
constexpr int OFF_Q = OFF_V + STAGES * KT * LDS * 2;             // [16][LDS] bf16
constexpr int OFF_KNEW = OFF_Q + ROWS * LDS * 2;                 // [LDS] bf16
constexpr int OFF_VNEW = OFF_KNEW + LDS * 2;                     // [LDS] bf16
constexpr int SMEM_TILES = OFF_VNEW + LDS * 2;
// After the key tiles are done their space is used again as the place where the cluster's blocks
// leave their results for this block's slice of the columns:
//   recv_o  [blocks of the cluster][WN warps][rows][columns of a slice] f32
//   recv_ml [blocks of the cluster][WN warps][rows][2] f32 (maximum, sum)
// `rows` = min(16, query heads per kv head); a slice is `cpo` column tiles of 8 (owner of column
// tile j: j / cpo, cpo = ceil(DT / blocks of the cluster)).
__host__ __device__ constexpr int slice_tiles(int csize) { return (DT + csize - 1) / csize; }
__host__ __device__ constexpr int recv_floats(int csize, int rows) {
    return csize * WN * rows * (slice_tiles(csize) * 8 + 2);
}
// shared memory of a launch: the tiles, or the receive area where that is larger (tiny heads)
static int smem_bytes_for(int rows) {
    int most = 0;
    for (int c = 1; c <= MAX_CLUSTER; ++c) most = most > recv_floats(c, rows) ? most : recv_floats(c, rows);
    const int recv = most * 4;
    return SMEM_TILES > recv ? SMEM_TILES : recv;
}

__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

#ifdef DECODE_TIMING
// Debugging aid, compiled on request only: wall-clock stamps of one block's phases.
__device__ unsigned long long decode_stamps[16];
#define STAMP(k)                                                                      \
    do {                                                                              \
        if (blockIdx.x == DECODE_TIMING && threadIdx.x == 0) {                        \
            unsigned long long t_;                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t_));                  \
            decode_stamps[k] = t_;                                                    \
        }                                                                             \
    } while (0)
#else
#define STAMP(k) do { } while (0)
#endif

__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ qkv, int qkv_stride,
                   __nv_bfloat16* __restrict__ out, int out_stride,
                   __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                   const int* __restrict__ block_table, int table_stride, int num_pages,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                   const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items, int cap,
                   float* __restrict__ partial_acc, float* __restrict__ partial_ml,
                   int* __restrict__ counters, const float* __restrict__ inv_freq, int rot,
                   int write_kv, int heads, int kv_heads, int page, float scale, int window,
                   int recv_rows, int* __restrict__ status) {
    (void)seq_slot;
    (void)seq_pos0;                    // both come with the items
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw + OFF_K);
    __nv_bfloat16* v_s = reinterpret_cast<__nv_bfloat16*>(smem_raw + OFF_V);
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw + OFF_Q);
    __nv_bfloat16* k_new = reinterpret_cast<__nv_bfloat16*>(smem_raw + OFF_KNEW);
    __nv_bfloat16* v_new = reinterpret_cast<__nv_bfloat16*>(smem_raw + OFF_VNEW);
    __shared__ int s_last;

    STAMP(0);
    DE_TRACE_EVENT(2, 0);
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int group = blockIdx.x / csize;                 // (items' cluster, kv head)
    const int hk = group % kv_heads;
    const int item_index = (group / kv_heads) * csize + rank;
    // the items of this kernel carry the token's position and its sequence's slot in place of
    // the partial slots (one dependent read less before the first copies can be requested)
    const WorkItem it = items[item_index];
    const bool empty = it.kv_begin >= it.kv_end;          // padding: takes part in the merge only
    const int g = heads / kv_heads;
    const int pos = it.partial;                           // the token's position
    const int slot = it.first_partial;
    const int tok = seq_qstart[it.seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wn = warp;
    const int gid = lane >> 2, tig = lane & 3;
    const int n_rows = min(ROWS, g - it.row0);
    // the tile's clusters: `cap` items a tile, csize of them a cluster
    const int clusters_per_tile = cap / csize;
    const int cluster_in_tile = (item_index - it.tile * cap) / csize;
    // the token's own key lies in this block's range and is not in the cache yet
    const bool new_key = !empty && write_kv != 0 && pos >= it.kv_begin && pos < it.kv_end;

    // every row is the same token: one key range
    int lo = it.kv_begin;
    if (window > 0) lo = max(lo, pos - window + 1);
    const int hi = empty ? lo : min(it.kv_end, pos + 1);
    const int k_lo = (lo / KT) * KT;

    const size_t slab = (size_t)page * D;
    // keys and values of a tile from the cache; the token's own row is left out (fill_new)
    // (two threads take a key's row, one look into the block table each; they alternate over
    // the row's 16-byte pieces, so that every request of the pair fills a whole 32-byte sector)
    static_assert(THREADS == 2 * KT && CHUNKS % 2 == 0, "two threads a key row");
    auto load_tile = [&](int kt, int stage) {
        __nv_bfloat16* kd = k_s + stage * KT * LDS;
        __nv_bfloat16* vd = v_s + stage * KT * LDS;
        const int j = threadIdx.x >> 1, ch0 = threadIdx.x & 1;
        const int kpos = kt + j;
        if (new_key && kpos == pos) return;
        bool ok = kpos >= lo && kpos < hi;
        size_t off = 0;
        if (ok) {
            const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
            ok = page_id >= 0 && page_id < num_pages;
            if (ok) off = ((size_t)page_id * kv_heads + hk) * slab + (size_t)(kpos % page) * D;
            else if (ch0 == 0) atomicExch(status, 2);                // a visible key has no page
        }
#pragma unroll
        for (int ch = ch0; ch < CHUNKS; ch += 2) {
            cp_async16(kd + j * LDS + ch * 8, k_pages + off + (ok ? ch * 8 : 0), ok);
            cp_async16(vd + j * LDS + ch * 8, v_pages + off + (ok ? ch * 8 : 0), ok);
        }
    };
    // the token's own key and value, from this launch and not from the cache, into their row
    auto fill_new = [&](int kt, int stage) {
        if (!new_key || pos < kt || pos >= kt + KT || threadIdx.x >= 2 * CHUNKS) return;
        const int ch = threadIdx.x % CHUNKS;
        __nv_bfloat16* dst = (threadIdx.x < CHUNKS ? k_s : v_s) + (stage * KT + pos - kt) * LDS;
        const __nv_bfloat16* src = threadIdx.x < CHUNKS ? k_new : v_new;
        *reinterpret_cast<uint4*>(dst + ch * 8) = *reinterpret_cast<const uint4*>(src + ch * 8);
    };

    // the first tiles are requested before the wait, unless this step's own key is among what
    // the cache is read for (see the head of the file)
    const bool early = write_kv != 0;
    if (early) {
#pragma unroll
        for (int t = 0; t < STAGES; ++t) {
            if (k_lo + t * KT < hi) load_tile(k_lo + t * KT, t);
            cp_async_commit();
        }
    }

    // what does not depend on qkv: the angles' cosines and sines, the page the token's key goes to
    const int half = rot / 2;
    constexpr int TODO = (ROWS + 1) * (D / 2);            // pairs of 16 q rows and of the key
    constexpr int PER = (TODO + THREADS - 1) / THREADS;
    // every row is the same token, so the angles depend on the pair's index alone
    __shared__ float cos_s[D / 2], sin_s[D / 2];
    for (int j = threadIdx.x; j < D / 2; j += THREADS) {
        const bool rotated = !empty && j < half && inv_freq != nullptr;
        const float angle = rotated ? (float)pos * inv_freq[j] : 0.0f;
        cos_s[j] = cosf(angle);
        sin_s[j] = sinf(angle);
    }
    int write_page = -1;
    if (new_key && it.row0 == 0 && threadIdx.x < 2 * CHUNKS)
        write_page = block_table[(size_t)slot * table_stride + pos / page];

    STAMP(1);
    pdl_wait();                                       // qkv is the previous kernel's output
    DE_TRACE_EVENT(2, 1);
    if (!early) {
#pragma unroll
        for (int t = 0; t < STAGES; ++t) {
            if (k_lo + t * KT < hi) load_tile(k_lo + t * KT, t);
            cp_async_commit();
        }
    }
    __syncthreads();                                  // the cosines and sines are in place
    STAMP(2);

    float o_acc[DT][4];
#pragma unroll
    for (int j = 0; j < DT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float sl = scale * 1.4426950408889634f;           // scores in the exp2 domain

    if (!empty) {
        // rotation (half-split pairs, angle = float(pos) * inv_freq[j]); features from `rot` on
        // stay.  Every thread first requests all it needs (independent loads), then computes.
        const __nv_bfloat16* token = qkv + (size_t)tok * qkv_stride;
        {
            __nv_bfloat16 a[PER], bb[PER];
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int idx = threadIdx.x + u * THREADS;
                const int r = idx / (D / 2), j = idx - r * (D / 2);
                const bool live = r < n_rows || (r == ROWS && new_key);
                const int c0 = j < half ? j : rot + 2 * (j - half);
                const int c1 = j < half ? j + half : c0 + 1;
                const __nv_bfloat16* src =
                    token + (size_t)(r < ROWS ? hk * g + it.row0 + r : heads + hk) * D;
                a[u] = live ? src[c0] : __float2bfloat16_rn(0.0f);
                bb[u] = live ? src[c1] : __float2bfloat16_rn(0.0f);
            }
            __nv_bfloat16 vn = __float2bfloat16_rn(0.0f);
            if (new_key && threadIdx.x < D)
                vn = token[(size_t)(heads + kv_heads + hk) * D + threadIdx.x];
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int idx = threadIdx.x + u * THREADS;
                const int r = idx / (D / 2), j = idx - r * (D / 2);
                if (r > ROWS || (r == ROWS && !new_key)) continue;
                __nv_bfloat16* dst = r < ROWS ? q_s + r * LDS : k_new;
                const int c0 = j < half ? j : rot + 2 * (j - half);
                const int c1 = j < half ? j + half : c0 + 1;
                if (j < half && inv_freq && (r < n_rows || r == ROWS)) {
                    float ra, rb;
                    rope_rotate(__bfloat162float(a[u]), __bfloat162float(bb[u]), cos_s[j], sin_s[j],
                                ra, rb);
                    dst[c0] = __float2bfloat16_rn(ra);
                    dst[c1] = __float2bfloat16_rn(rb);
                } else {                              // unrotated features; zeros beyond the group
                    dst[c0] = a[u];
                    dst[c1] = bb[u];
                }
            }
            if (new_key) {
                if (threadIdx.x < D) v_new[threadIdx.x] = vn;
                for (int j = threadIdx.x + THREADS; j < D; j += THREADS)
                    v_new[j] = token[(size_t)(heads + kv_heads + hk) * D + j];
            }
        }
        __syncthreads();

        // the token's key and value into the cache: the block of the group's first rows does it
        if (new_key && it.row0 == 0 && threadIdx.x < 2 * CHUNKS) {
            if (write_page < 0 || write_page >= num_pages) {  // no page here: record, skip
                if (threadIdx.x == 0) atomicExch(status, 1);
            } else {
                const size_t off =
                    ((size_t)write_page * kv_heads + hk) * page * D + (size_t)(pos % page) * D;
                const int ch = threadIdx.x % CHUNKS;
                if (threadIdx.x < CHUNKS)
                    *reinterpret_cast<uint4*>(k_pages + off + ch * 8) =
                        *reinterpret_cast<const uint4*>(k_new + ch * 8);
                else
                    *reinterpret_cast<uint4*>(v_pages + off + ch * 8) =
                        *reinterpret_cast<const uint4*>(v_new + ch * 8);
            }
        }
#pragma unroll
        for (int t = 0; t < STAGES; ++t) fill_new(k_lo + t * KT, t);
        STAMP(3);

        unsigned qf[D / 16][4];
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat16* p = q_s + (gid + 8 * i) * LDS + kk * 16 + 2 * tig;
                qf[kk][i] = *reinterpret_cast<const unsigned*>(p);
                qf[kk][i + 2] = *reinterpret_cast<const unsigned*>(p + 8);
            }

        int stage = 0;
        for (int kt = k_lo; kt < hi; kt += KT, stage = stage + 1 == STAGES ? 0 : stage + 1) {
            cp_async_wait<STAGES - 1>();              // this tile has landed; the next may be on their way
            __syncthreads();

            const __nv_bfloat16* kb = k_s + stage * KT * LDS + wn * NK * LDS;
            const __nv_bfloat16* vb = v_s + stage * KT * LDS + wn * NK * LDS;

            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    unsigned b[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4(b, kb + ((j + (mat >> 1)) * 8 + r) * LDS + kk * 16 + (mat & 1) * 8);
                    mma_bf16(s[j], qf[kk], b[0], b[1]);
                    mma_bf16(s[j + 1], qf[kk], b[2], b[3]);
                }
            }
            const int key0 = kt + wn * NK;
            if (key0 + NK > hi || key0 < lo) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + 2 * tig + (e & 1);
                        if (key < lo || key >= hi) s[j][e] = -INFINITY;
                    }
            }

            unsigned pf[NK / 16][4];
            {
                float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    m_new[0] = fmaxf(m_new[0], fmaxf(s[j][0], s[j][1]));
                    m_new[1] = fmaxf(m_new[1], fmaxf(s[j][2], s[j][3]));
                }
                float corr[2], m_use[2], l_add[2] = {0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
                    m_use[i] = m_new[i] == -INFINITY ? 0.0f : m_new[i];
                    corr[i] = fast_exp2((m_run[i] - m_use[i]) * sl);
                    m_run[i] = m_new[i];
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const float p0 = fast_exp2((s[j][0] - m_use[0]) * sl);
                    const float p1 = fast_exp2((s[j][1] - m_use[0]) * sl);
                    const float p2 = fast_exp2((s[j][2] - m_use[1]) * sl);
                    const float p3 = fast_exp2((s[j][3] - m_use[1]) * sl);
                    l_add[0] += p0 + p1;
                    l_add[1] += p2 + p3;
                    pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                    pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
                for (int j = 0; j < DT; ++j) {
                    o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
                    o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
                }
            }
#pragma unroll
            for (int ks = 0; ks < NK / 16; ++ks) {
#pragma unroll
                for (int jd = 0; jd < DT; jd += 2) {
                    unsigned b[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4_trans(b, vb + (ks * 16 + (mat & 1) * 8 + r) * LDS +
                                             (jd + (mat >> 1)) * 8);
                    mma_bf16(o_acc[jd], pf[ks], b[0], b[1]);
                    mma_bf16(o_acc[jd + 1], pf[ks], b[2], b[3]);
                }
            }
            __syncthreads();                   // this stage is free: the tile after the next goes there
            if (kt + STAGES * KT < hi) {
                load_tile(kt + STAGES * KT, stage);
                fill_new(kt + STAGES * KT, stage);
            }
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    STAMP(4);
    pdl_trigger();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }

    // ---- every block of the cluster is through its tiles: their space is free everywhere
    STAMP(5);
    DE_TRACE_EVENT(2, 3);
    cluster_arrive();
    cluster_wait();
    DE_TRACE_EVENT(2, 4);
    STAMP(6);
    const int cpo = slice_tiles(csize);                        // column tiles of a slice
    const int ld_o = cpo * 8;
    float* recv_o = reinterpret_cast<float*>(smem_raw);
    float* recv_ml = recv_o + (size_t)csize * WN * recv_rows * ld_o;
    // ---- every warp leaves its result with the owners of the columns, from its registers
    {
        const int src = rank * WN + wn;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = gid + 8 * i;
            if (r >= n_rows) continue;
            for (int owner = tig; owner < csize; owner += 4)      // the row's maximum and sum
                *reinterpret_cast<float2*>(cluster.map_shared_rank(recv_ml, owner) +
                                           ((size_t)src * recv_rows + r) * 2) =
                    make_float2(m_run[i], l_run[i]);
            if (empty) continue;                                   // maximum -inf: nothing to add
#pragma unroll
            for (int j = 0; j < DT; ++j) {
                const int owner = j / cpo, jj = j - owner * cpo;
                *reinterpret_cast<float2*>(cluster.map_shared_rank(recv_o, owner) +
                                           ((size_t)src * recv_rows + r) * ld_o + jj * 8 + 2 * tig) =
                    make_float2(o_acc[j][2 * i], o_acc[j][2 * i + 1]);
            }
        }
    }
    cluster_arrive();
    cluster_wait();
    DE_TRACE_EVENT(2, 5);
    STAMP(7);
    // ---- the slice of this block, merged from its own shared memory
    const bool final_here = clusters_per_tile == 1;
    const size_t part_slot = (size_t)it.tile * clusters_per_tile + cluster_in_tile;
    __nv_bfloat16* out_token = out + (size_t)tok * out_stride + (size_t)(hk * g + it.row0) * D;
    const int col0 = rank * ld_o;                               // first column of the slice
    const int my_cols = max(0, min(D - col0, ld_o));
    const int sources = csize * WN;
    // with many sources (clusters of 4 blocks and more) four neighbouring lanes share a pair of
    // outputs: each merges a quarter of the sources (source p belongs to lane p % 4; there are
    // 4 x blocks of them), then the four merge theirs; with few, a lane takes all of them
    static_assert(WN == 4, "a quarter of the sources a lane");
    const int share = sources >= 16 ? 4 : 1;
    for (int idx = threadIdx.x; idx < n_rows * (my_cols / 2) * share; idx += THREADS) {
        const int e = share == 4 ? idx >> 2 : idx, quarter = share == 4 ? idx & 3 : 0;
        const int r = e / (my_cols / 2), dd = 2 * (e - r * (my_cols / 2));
        float m = -INFINITY;
        for (int p = quarter; p < sources; p += share)
            m = fmaxf(m, recv_ml[((size_t)p * recv_rows + r) * 2]);
        float l = 0.0f;
        float2 acc = make_float2(0.0f, 0.0f);
        for (int p = quarter; p < sources; p += share) {
            const float2 ml = *reinterpret_cast<const float2*>(recv_ml +
                                                               ((size_t)p * recv_rows + r) * 2);
            if (ml.x == -INFINITY) continue;                  // no visible key there
            const float f = fast_exp2((ml.x - m) * sl);
            const float2 v = *reinterpret_cast<const float2*>(
                recv_o + ((size_t)p * recv_rows + r) * ld_o + dd);
            l += ml.y * f;
            acc.x = fmaf(v.x, f, acc.x);
            acc.y = fmaf(v.y, f, acc.y);
        }
        if (share == 4) {
            const unsigned group = __activemask();            // (whole groups of four lanes)
            float m_all = fmaxf(m, __shfl_xor_sync(group, m, 1));
            m_all = fmaxf(m_all, __shfl_xor_sync(group, m_all, 2));
            const float mine = m == -INFINITY ? 0.0f : fast_exp2((m - m_all) * sl);
            l *= mine; acc.x *= mine; acc.y *= mine;
#pragma unroll
            for (int o = 1; o < 4; o <<= 1) {
                l += __shfl_xor_sync(group, l, o);
                acc.x += __shfl_xor_sync(group, acc.x, o);
                acc.y += __shfl_xor_sync(group, acc.y, o);
            }
            m = m_all;
            if (quarter != 0) continue;
        }
        if (final_here) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            *reinterpret_cast<unsigned*>(out_token + r * D + col0 + dd) =
                pack_bf16(acc.x * inv, acc.y * inv);
        } else {
            const size_t idx_p = (part_slot * kv_heads + hk) * ROWS + r;
            *reinterpret_cast<float2*>(partial_acc + idx_p * D + col0 + dd) = acc;
            if (col0 + dd == 0) {
                partial_ml[idx_p * 2] = m * scale;            // natural-log domain, as merged
                partial_ml[idx_p * 2 + 1] = l;
            }
        }
    }
    STAMP(8);
    DE_TRACE_EVENT(2, 2);
    if (final_here) return;

    // ---- several clusters a tile: the block that finishes last merges their partial results, in
    // ascending order of the chunks.  Clusters of padding only do not count and are not counted on.
    const int live_clusters = (it.chunks + csize - 1) / csize;
    if (cluster_in_tile >= live_clusters) return;
    __threadfence();                                   // this block's slice of the partial result
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = counters + (size_t)it.tile * kv_heads + hk;
        const int before = atomicAdd(counter, 1);
        s_last = before == live_clusters * csize - 1;
        if (s_last) *counter = 0;                    // as the next launch expects it
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t step = (size_t)kv_heads * ROWS;                   // from one slot to the next
    const size_t row0_idx = ((size_t)it.tile * clusters_per_tile * kv_heads + hk) * ROWS;
    for (int e = threadIdx.x; e < n_rows * D; e += THREADS) {
        const int r = e / D, dd = e - r * D;
        const size_t idx0 = row0_idx + r;
        float m = -INFINITY;
        for (int c0 = 0; c0 < live_clusters; c0 += 4) {
            float mm[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                mm[u] = c0 + u < live_clusters ? __ldcg(partial_ml + (idx0 + (c0 + u) * step) * 2)
                                               : -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; ++u) m = fmaxf(m, mm[u]);
        }
        float l = 0.0f, acc = 0.0f;
        for (int c0 = 0; c0 < live_clusters; c0 += 4) {
            float2 ml[4];
            float pa[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {              // independent loads: four chunks in flight
                const bool have = c0 + u < live_clusters;
                const size_t idx = idx0 + (c0 + u) * step;
                ml[u] = have ? __ldcg(reinterpret_cast<const float2*>(partial_ml) + idx)
                             : make_float2(-INFINITY, 0.0f);
                pa[u] = have ? __ldcg(partial_acc + idx * D + dd) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (ml[u].x == -INFINITY) continue;   // the chunk held no visible key
                const float f = expf(ml[u].x - m);
                l += ml[u].y * f;
                acc = fmaf(pa[u], f, acc);
            }
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        out_token[r * D + dd] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

#ifdef DECODE_TIMING
DE_EXPORT int de_attn_decode_stamps(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, decode_stamps, sizeof(decode_stamps));
}
#endif
DE_EXPORT int de_attn_decode_head_dim() { return D; }
DE_EXPORT int de_attn_decode_max_cluster() { return MAX_CLUSTER; }
// Blocks of the kernel that an SM holds at once (registers and shared memory), or 0 if unknown.
// (`group`: query heads per kv head; the receive area of the merge grows with it for tiny heads)
DE_EXPORT int de_attn_decode_blocks_per_sm(int group) {
    const int smem = smem_bytes_for(group < ROWS ? group : ROWS);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem) != cudaSuccess)
        return 0;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_kernel, THREADS, smem) !=
        cudaSuccess)
        return 0;
    return n;
}

// `items`: tiles x `cap` work items (see the head of the file), `cluster` blocks a cluster (1 to 8;
// `cap` a multiple of it).  `partial_acc` / `partial_ml`: room for tiles * cap / cluster
// partial results (each kv_heads x 16 rows), used when cap > cluster.  `counters`: int32, one per
// (tile, kv head), zero before the first launch.  `inv_freq` null: no rotation.  `write_kv` 0: the
// layer reads a cache that an earlier layer of the step wrote, the token's key included.
DE_EXPORT int de_attn_decode(const void* qkv, int qkv_stride, void* out, int out_stride,
                             void* k_pages, void* v_pages, const int* block_table,
                             int table_stride, int num_pages, const int* seq_slot,
                             const int* seq_qstart, const int* seq_pos0, const int* items,
                             int num_items, int cap, int cluster, float* partial_acc,
                             float* partial_ml, int* counters, const float* inv_freq, int rot,
                             int write_kv, int heads, int kv_heads, int head_dim, int page,
                             float scale, int window, int* status, void* stream) {
    if (num_items <= 0) return 0;
    if (head_dim != D || heads % kv_heads != 0) return -2;
    if (rot < 0 || rot > D || (rot & 1)) return -2;
    if (cluster < 1 || cluster > MAX_CLUSTER || cap < cluster || cap % cluster != 0 ||
        num_items % cap != 0)
        return -4;
    if (cap > cluster && (partial_acc == nullptr || partial_ml == nullptr)) return -4;
    // 16-byte rows of keys and values
    if (qkv_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)qkv & 15) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return -3;
    const int recv_rows = heads / kv_heads < ROWS ? heads / kv_heads : ROWS;
    const int SMEM_BYTES = smem_bytes_for(recv_rows);
    if (SMEM_BYTES > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
    }
    // the step's common split of an SM's memory, unless this launch needs more blocks an SM than
    // that leaves room for (then the driver's choice for this kernel)
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    const long long blocks = (long long)num_items * kv_heads;
    // (the split is rounded up to one of these sizes; a block takes 1 KB beside its own)
    const int sizes_kb[] = {8, 16, 32, 64, 100, 132, 164, 196, 228};
    int split_kb = 228;
    for (int i = 8; i >= 0; --i)
        if (sizes_kb[i] * 100 >= g_carveout * 228) split_kb = sizes_kb[i];
    const long long room = g_carveout < 0 ? 0 : (long long)split_kb * 1024 / (SMEM_BYTES + 1024);
    // (one block an SM fewer than fit: clusters need their blocks placed together, and a launch
    // that fills every place waits for places; measured at batch 12, 384 blocks of 444 places)
    de_prefer_carveout(attn_decode_kernel, blocks <= (room - 1) * sms ? g_carveout : -1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)num_items * (unsigned)kv_heads);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 2 : 1;
    return de_check(cudaLaunchKernelEx(
        &cfg, attn_decode_kernel, (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)out,
        out_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_stride,
        num_pages, seq_slot, seq_qstart, seq_pos0, (const WorkItem*)items, cap, partial_acc,
        partial_ml, counters, inv_freq, rot, write_kv, heads, kv_heads, page, scale, window,
        recv_rows, status));
}
