// Attention over the paged cache on the tensor cores, bfloat16 operands, float32 accumulation and
// softmax.  Compiled once per head size (-DHEAD_DIM=d, d a multiple of 16 up to 256), so a run
// compiles the head size of its model only.
//
// The same work items as the float32 kernel (attention_simt.cu): a tile of query rows of one
// sequence and one kv head, rows being (token, query head in the kv head's group), with a range of
// key positions; grouped-query heads share every key/value tile that is loaded
// (the reference expands k and v in memory instead, src/layers/attention.py:35-36).
// Two shapes of one kernel body:
//   wide   - 64 rows: 4 warps x 16 rows, every warp sees all 64 keys of a tile (prompt portions);
//   narrow - 16 rows: 4 warps split the 64 keys of a tile among them and merge at the end
//            (decoded tokens: few rows, long key ranges).
// Keys and values come from the pages through the block table with cp.async (16 bytes a copy,
// zero fill outside the item's range), two tiles in flight; q k^T and p v are mma.sync m16n8k16;
// the softmax is the running maximum / sum form in float32 (exp2 with the scale folded in), masks
// as in src/layers/attention.py:41-64 plus an optional window.  An item that covers a chunk of a
// long key range writes an unnormalised partial (accumulator, maximum, sum) in the layout that
// `de_attn_combine` merges.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

#include "attention_mma_common.cuh"

namespace {

// WM warps along the rows, WN warps along the keys of a tile; WM * WN = 4.  Each warp owns RT
// m16 row tiles (16 RT rows) that share every key/value fragment it reads from shared memory:
// with RT = 2 a fragment feeds two mma instructions, which halves the shared-memory traffic per
// flop (the wide shape is bound by it).
template <int WM, int WN, int RT>
__global__ void __launch_bounds__(THREADS)
attn_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                int table_stride, int num_pages, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items,
                float* __restrict__ partial_acc, float* __restrict__ partial_ml, int heads,
                int kv_heads, int page, float scale, int window, int* __restrict__ status) {
    static_assert(WN == 1 || RT == 1, "warps that split the keys own one row tile");
    constexpr int ROWS = WM * 16 * RT;     // rows of the tile
    constexpr int NK = KT / WN;            // keys of a tile that one warp sees
    constexpr int NT = NK / 8;             // score tiles (n = 8) per warp
    constexpr int DT = D / 8;              // output tiles (n = 8)
    constexpr int CHUNKS = D / 8;          // 16-byte copies in one key's row
    constexpr int R2 = 2 * RT;             // rows of one thread

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [2][KT][LDS]
    __nv_bfloat16* v_s = k_s + 2 * KT * LDS;                                  // [2][KT][LDS]

    // blocks are numbered item-major, so that the items run in the order the host gave them
    const WorkItem it = items[blockIdx.x / kv_heads];
    if (it.kv_begin >= it.kv_end) {                                           // padding item
        pdl_wait();
        return;
    }
    const int hk = blockIdx.x % kv_heads;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp / WN, wn = warp % WN;
    const int gid = lane >> 2, tig = lane & 3;

    // the rows of this thread: gid and gid + 8 of each of the warp's row tiles
    int row[R2], pos[R2], tok[R2], hq[R2];
    bool live[R2];
#pragma unroll
    for (int r = 0; r < R2; ++r) {
        row[r] = it.row0 + (wm * RT + (r >> 1)) * 16 + gid + 8 * (r & 1);
        live[r] = row[r] < rows_total;
        tok[r] = live[r] ? row[r] / g : 0;
        hq[r] = hk * g + (live[r] ? row[r] % g : 0);
        pos[r] = live[r] ? pos0 + tok[r] : -1;
    }

    pdl_wait();            // q, and the keys and values of this step's tokens, are just written

    // q fragments straight from global memory (read once)
    unsigned qf[RT][D / 16][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = 2 * rt + i;
                const __nv_bfloat16* p = q + (size_t)(tok0 + tok[r]) * q_stride + hq[r] * D +
                                         kk * 16 + 2 * tig;
                qf[rt][kk][i] = live[r] ? *reinterpret_cast<const unsigned*>(p) : 0u;
                qf[rt][kk][i + 2] = live[r] ? *reinterpret_cast<const unsigned*>(p + 8) : 0u;
            }

    // key range of the tile and of this thread's rows
    const int last_row = min(it.row0 + ROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    int k_lo_true = it.kv_begin;
    if (window > 0) k_lo_true = max(k_lo_true, min_pos - window + 1);
    const int k_lo = (k_lo_true / KT) * KT;
    int lo[R2], hi[R2];
    int min_hi = 0x7fffffff, max_lo = 0;
#pragma unroll
    for (int r = 0; r < R2; ++r) {
        lo[r] = it.kv_begin;
        if (window > 0) lo[r] = max(lo[r], pos[r] - window + 1);
        hi[r] = min(it.kv_end, pos[r] + 1);          // pos -1 (dead row): nothing is visible
        min_hi = min(min_hi, hi[r]);
        max_lo = max(max_lo, lo[r]);
    }
    // over the warp: is every key of a tile visible to every row?  (rows differ per lane)
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        min_hi = min(min_hi, __shfl_xor_sync(0xffffffffu, min_hi, o));
        max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, o));
    }

    const size_t slab = (size_t)page * D;
    auto load_tile = [&](int kt, int stage) {
        __nv_bfloat16* kd = k_s + stage * KT * LDS;
        __nv_bfloat16* vd = v_s + stage * KT * LDS;
        for (int c = threadIdx.x; c < KT * CHUNKS; c += THREADS) {
            const int j = c / CHUNKS, ch = c - j * CHUNKS;
            const int kpos = kt + j;
            bool ok = kpos >= k_lo_true && kpos < k_hi;
            size_t off = 0;
            if (ok) {
                const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
                ok = page_id >= 0 && page_id < num_pages;
                if (ok) off = ((size_t)page_id * kv_heads + hk) * slab + (size_t)(kpos % page) * D +
                              ch * 8;
                else if (status != nullptr) atomicExch(status, 2);   // a visible key has no page
            }
            cp_async16(kd + j * LDS + ch * 8, k_pages + off, ok);
            cp_async16(vd + j * LDS + ch * 8, v_pages + off, ok);
        }
    };

    float o_acc[RT][DT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int j = 0; j < DT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o_acc[rt][j][e] = 0.0f;
    float m_run[R2], l_run[R2];
#pragma unroll
    for (int r = 0; r < R2; ++r) { m_run[r] = -INFINITY; l_run[r] = 0.0f; }
    const float sl = scale * 1.4426950408889634f;           // scores in the exp2 domain

    load_tile(k_lo, 0);
    cp_async_commit();
    int stage = 0;
    for (int kt = k_lo; kt < k_hi; kt += KT, stage ^= 1) {
        if (kt + KT < k_hi) load_tile(kt + KT, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const __nv_bfloat16* kb = k_s + stage * KT * LDS + wn * NK * LDS;
        const __nv_bfloat16* vb = v_s + stage * KT * LDS + wn * NK * LDS;

        // s = q k^T : 16 RT rows x NK keys
        float s[RT][NT][4];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[rt][j][e] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                unsigned b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, kb + ((j + (mat >> 1)) * 8 + r) * LDS + kk * 16 + (mat & 1) * 8);
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    mma_bf16(s[rt][j], qf[rt][kk], b[0], b[1]);
                    mma_bf16(s[rt][j + 1], qf[rt][kk], b[2], b[3]);
                }
            }
        }

        // masks (only on tiles that reach a limit)
        const int key0 = kt + wn * NK;
        if (key0 + NK > min_hi || key0 < max_lo) {
#pragma unroll
            for (int rt = 0; rt < RT; ++rt)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + 2 * tig + (e & 1);
                        const int r = 2 * rt + (e >> 1);
                        if (key < lo[r] || key >= hi[r]) s[rt][j][e] = -INFINITY;
                    }
        }

        // running softmax
        unsigned pf[RT][NK / 16][4];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
            float m_new[2] = {m_run[2 * rt], m_run[2 * rt + 1]};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                m_new[0] = fmaxf(m_new[0], fmaxf(s[rt][j][0], s[rt][j][1]));
                m_new[1] = fmaxf(m_new[1], fmaxf(s[rt][j][2], s[rt][j][3]));
            }
            float corr[2], m_use[2], l_add[2] = {0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
                m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
                m_use[i] = m_new[i] == -INFINITY ? 0.0f : m_new[i];
                corr[i] = fast_exp2((m_run[2 * rt + i] - m_use[i]) * sl);   // 0 while m_run is -inf
                m_run[2 * rt + i] = m_new[i];
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const float p0 = fast_exp2((s[rt][j][0] - m_use[0]) * sl);
                const float p1 = fast_exp2((s[rt][j][1] - m_use[0]) * sl);
                const float p2 = fast_exp2((s[rt][j][2] - m_use[1]) * sl);
                const float p3 = fast_exp2((s[rt][j][3] - m_use[1]) * sl);
                l_add[0] += p0 + p1;
                l_add[1] += p2 + p3;
                pf[rt][j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                pf[rt][j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
                l_run[2 * rt + i] = l_run[2 * rt + i] * corr[i] + l_add[i];
#pragma unroll
            for (int j = 0; j < DT; ++j) {
                o_acc[rt][j][0] *= corr[0]; o_acc[rt][j][1] *= corr[0];
                o_acc[rt][j][2] *= corr[1]; o_acc[rt][j][3] *= corr[1];
            }
        }

        // o += p v
#pragma unroll
        for (int ks = 0; ks < NK / 16; ++ks) {
#pragma unroll
            for (int jd = 0; jd < DT; jd += 2) {
                unsigned b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vb + (ks * 16 + (mat & 1) * 8 + r) * LDS +
                                         (jd + (mat >> 1)) * 8);
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    mma_bf16(o_acc[rt][jd], pf[rt][ks], b[0], b[1]);
                    mma_bf16(o_acc[rt][jd + 1], pf[rt][ks], b[2], b[3]);
                }
            }
        }
        __syncthreads();                       // this stage may be overwritten by the next load
    }
    cp_async_wait<0>();
    pdl_trigger();

    // row sums live in the 4 lanes of a quad
#pragma unroll
    for (int r = 0; r < R2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }

    if constexpr (WN == 1) {
#pragma unroll
        for (int r = 0; r < R2; ++r) {
            if (!live[r]) continue;
            const int rt = r >> 1, i = r & 1;
            if (it.partial < 0) {
                const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
                __nv_bfloat16* o = out + (size_t)(tok0 + tok[r]) * out_stride + hq[r] * D;
#pragma unroll
                for (int j = 0; j < DT; ++j)
                    *reinterpret_cast<unsigned*>(o + j * 8 + 2 * tig) =
                        pack_bf16(o_acc[rt][j][2 * i] * inv, o_acc[rt][j][2 * i + 1] * inv);
            } else {
                const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + (row[r] - it.row0);
                float* pa = partial_acc + idx * D;
#pragma unroll
                for (int j = 0; j < DT; ++j) {
                    pa[j * 8 + 2 * tig] = o_acc[rt][j][2 * i];
                    pa[j * 8 + 2 * tig + 1] = o_acc[rt][j][2 * i + 1];
                }
                if (tig == 0) {
                    partial_ml[idx * 2] = m_run[r] * scale;      // natural-log domain, as merged
                    partial_ml[idx * 2 + 1] = l_run[r];
                }
            }
        }
    } else {
        // merge the WN warps that split the keys: through shared memory (the tiles are done)
        float* red_o = reinterpret_cast<float*>(smem_raw);             // [WN][16][D]
        float* red_m = red_o + WN * 16 * D;                             // [WN][16]
        float* red_l = red_m + WN * 16;                                 // [WN][16]
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = gid + 8 * i;
            float* dst = red_o + ((size_t)wn * 16 + r) * D;
#pragma unroll
            for (int j = 0; j < DT; ++j) {
                dst[j * 8 + 2 * tig] = o_acc[0][j][2 * i];
                dst[j * 8 + 2 * tig + 1] = o_acc[0][j][2 * i + 1];
            }
            if (tig == 0) {
                red_m[wn * 16 + r] = m_run[i];
                red_l[wn * 16 + r] = l_run[i];
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 16 * D; e += THREADS) {
            const int r = e / D, dd = e - r * D;
            const int rr = it.row0 + r;
            if (rr >= rows_total) continue;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < WN; ++w) m = fmaxf(m, red_m[w * 16 + r]);
            float l = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WN; ++w) {
                const float mw = red_m[w * 16 + r];
                if (mw == -INFINITY) continue;
                const float f = exp2f((mw - m) * sl);
                l += red_l[w * 16 + r] * f;
                acc += red_o[((size_t)w * 16 + r) * D + dd] * f;
            }
            if (it.partial < 0) {
                const int t = rr / g, h = hk * g + rr % g;
                out[(size_t)(tok0 + t) * out_stride + h * D + dd] =
                    __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
            } else {
                const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + r;
                partial_acc[idx * D + dd] = acc;
                if (dd == 0) {
                    partial_ml[idx * 2] = m * scale;
                    partial_ml[idx * 2 + 1] = l;
                }
            }
        }
    }
}

constexpr int WIDE_RT = D <= 64 ? 2 : 1;       // row tiles per warp of the wide shape

template <int WM, int WN, int RT>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
           const void* v_pages, const int* block_table, int table_stride, int num_pages,
           const int* seq_slot, const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
           const int* items, int num_items, float* partial_acc, float* partial_ml, int heads,
           int kv_heads, int page, float scale, int window, int* status, cudaStream_t s) {
    size_t smem = (size_t)4 * KT * LDS * sizeof(__nv_bfloat16);
    const size_t red = (size_t)WN * 16 * (D + 2) * sizeof(float);
    if (WN > 1 && red > smem) smem = red;
    auto kernel = attn_mma_kernel<WM, WN, RT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)num_items * (unsigned)kv_heads);
    return de_launch(kernel, grid, dim3(THREADS), smem, s, (const __nv_bfloat16*)q, q_stride,
                     (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages,
                     (const __nv_bfloat16*)v_pages, block_table, table_stride, num_pages, seq_slot,
                     seq_qstart, seq_qlen, seq_pos0, (const WorkItem*)items, partial_acc,
                     partial_ml, heads, kv_heads, page, scale, window, status);
}

}  // namespace

DE_EXPORT int de_attn_mma_head_dim() { return D; }

// rows of a tile of each shape (the host plans with these)
DE_EXPORT int de_attn_mma_rows(int shape) { return shape == 0 ? 4 * 16 * WIDE_RT : 16; }

// shape 0: wide (64 or 128 rows a tile), shape 1: narrow (16 rows a tile)
DE_EXPORT int de_attn_mma(int shape, const void* q, int q_stride, void* out, int out_stride,
                          const void* k_pages, const void* v_pages, const int* block_table,
                          int table_stride, int num_pages, const int* seq_slot,
                          const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                          const int* items, int num_items, float* partial_acc, float* partial_ml,
                          int heads, int kv_heads, int head_dim, int page, float scale, int window,
                          int* status, void* stream) {
    if (num_items <= 0) return 0;
    if (head_dim != D || heads % kv_heads != 0) return -2;
    if (q_stride % 2 != 0 || out_stride % 2 != 0) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (shape == 0)
        return launch<4, 1, WIDE_RT>(q, q_stride, out, out_stride, k_pages, v_pages, block_table,
                            table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0, items,
                            num_items, partial_acc, partial_ml, heads, kv_heads, page, scale, window,
                            status, s);
    return launch<1, 4, 1>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                        num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0, items, num_items,
                        partial_acc, partial_ml, heads, kv_heads, page, scale, window, status, s);
}

