// Element-wise and row-wise kernels of the step: embedding rows, residual sum + RMS norm,
// position rotation + write into the paged cache, silu(gate)*up, arg-max and temperature sampling.
// Every kernel exists for float32 and for bfloat16 storage; the arithmetic is float32 in both.
//
// What they replace in the reference (library calls there): F.embedding
// (src/layers/embed_head.py:13), the RMS norm (src/layers/layernorm.py:12-23) and the residual
// sums (src/models/llama.py:74-89), the rotation (src/layers/rotary_embedding.py:29-54), the
// per-token cache writes (src/distengine/paged_kv_cache.py:162-175,311-312), silu*up
// (src/layers/activation.py:8-9) and arg-max (src/layers/sampler.py:8).

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

// ------------------------------------------------------------------------------------------
// embedding: out[n, :] = float(table[ids[n], :])           (the residual stream starts here)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                  float* __restrict__ out, int width, int vocab) {
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 || id >= vocab) id = 0;          // ids are validated on the host; never read outside
    const T* row = table + (size_t)id * width;
    float* dst = out + (size_t)n * width;
    pdl_wait();                                  // the last step's kernels may still read `out`
    pdl_trigger();
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(row[i]);
}

DE_EXPORT int de_embed_rows(int dtype, const int* ids, const void* table, float* out, int n,
                            int width, int vocab, void* stream) {
    if (n <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16)
        return de_launch(embed_rows_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s, ids,
                         (const __nv_bfloat16*)table, out, width, vocab);
    return de_launch(embed_rows_kernel<float>, dim3(n), dim3(threads), 0, s, ids,
                     (const float*)table, out, width, vocab);
}

// ------------------------------------------------------------------------------------------
// residual sum + RMS norm.
//   x = resid[row] (+ delta[row]);  resid[row] = x (when update);  var = mean(x^2)
//   y = T(x * rsqrt(var + eps));    out[i] = T(float(y) * float(weight))
// The cast to the activation type comes before the multiplication by the weight, as in
// src/layers/layernorm.py:21-23.  `rows` (may be null) picks the rows to normalise: out[i] comes
// from row rows[i], and resid is then left as it is.
// ------------------------------------------------------------------------------------------
template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps) {
    __shared__ float scratch[33];
    const int i_out = blockIdx.x;
    const int row = rows ? rows[i_out] : i_out;
    float* r = resid + (size_t)row * width;
    const T* d = delta ? delta + (size_t)row * width : nullptr;
    const bool update = (rows == nullptr) && (delta != nullptr);
    pdl_wait();

    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = r[i];
        if (d) x += to_float(d[i]);
        if (update) r[i] = x;
        ss += x * x;
    }
    const float total = block_sum(ss, scratch);
    pdl_trigger();
    const float inv = rsqrtf(total / (float)width + eps);
    T* o = out + (size_t)i_out * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = r[i];
        if (d && !update) x += to_float(d[i]);       // same sum as above, bit for bit
        const float y = to_float(from_float<T>(x * inv));
        o[i] = from_float<T>(y * to_float(weight[i]));
    }
}

// four consecutive elements as one load or store
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const unsigned*>(&a);
        t.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

// The same for widths that are a multiple of 4 and at most 4 * CHUNKS * blockDim: the row stays in
// registers between the sum of squares and the scaling, every access is 8 or 16 bytes wide.
template <typename T, typename W, int CHUNKS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const W* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int width, float eps) {
    __shared__ float scratch[33];
    const int i_out = blockIdx.x;
    const int row = rows ? rows[i_out] : i_out;
    float* r = resid + (size_t)row * width;
    const T* d = delta ? delta + (size_t)row * width : nullptr;
    const bool update = (rows == nullptr) && (delta != nullptr);
    const int quads = width >> 2;

    float wv[CHUNKS][4];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {               // the weight is no kernel's output
        const int qd = threadIdx.x + c * blockDim.x;
        if (qd < quads) Vec4<W>::load(weight + 4 * qd, wv[c]);
    }
    pdl_wait();

    float x[CHUNKS][4];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int qd = threadIdx.x + c * blockDim.x;
        if (qd < quads) {
            Vec4<float>::load(r + 4 * qd, x[c]);
            if (d) {
                float dv[4];
                Vec4<T>::load(d + 4 * qd, dv);
#pragma unroll
                for (int e = 0; e < 4; ++e) x[c][e] += dv[e];
            }
            if (update) Vec4<float>::store(r + 4 * qd, x[c]);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += x[c][e] * x[c][e];
        }
    }
    const float total = block_sum(ss, scratch);
    pdl_trigger();
    const float inv = rsqrtf(total / (float)width + eps);
    T* o = out + (size_t)i_out * width;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int qd = threadIdx.x + c * blockDim.x;
        if (qd < quads) {
            float y[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                y[e] = to_float(from_float<T>(x[c][e] * inv)) * wv[c][e];
            Vec4<T>::store(o + 4 * qd, y);
        }
    }
}

template <typename T, typename W>
static int launch_add_rmsnorm(float* resid, const void* delta, const void* weight, void* out,
                              const int* rows, int n_out, int width, float eps, cudaStream_t s) {
    const bool aligned = width % 4 == 0 && ((uintptr_t)resid % 16 == 0) &&
                         ((uintptr_t)delta % 8 == 0) && ((uintptr_t)weight % 16 == 0) &&
                         ((uintptr_t)out % 16 == 0);
    const int quads = width / 4;
#define VEC(CH, TH)                                                                           \
    return de_launch(add_rmsnorm_vec_kernel<T, W, CH>, dim3(n_out), dim3(TH), 0, s, resid,    \
                     (const T*)delta, (const W*)weight, (T*)out, rows, width, eps)
    if (aligned && quads <= 128) VEC(1, 128);
    if (aligned && quads <= 256) VEC(1, 256);
    if (aligned && quads <= 512) VEC(2, 256);
    if (aligned && quads <= 1024) VEC(4, 256);
    if (aligned && quads <= 2048) VEC(4, 512);
    if (aligned && quads <= 4096) VEC(8, 512);
#undef VEC
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    return de_launch(add_rmsnorm_kernel<T, W>, dim3(n_out), dim3(threads), 0, s, resid,
                     (const T*)delta, (const W*)weight, (T*)out, rows, width, eps);
}

DE_EXPORT int de_add_rmsnorm(int dtype, int weight_dtype, float* resid, const void* delta,
                             const void* weight, void* out, const int* rows, int n_out, int width,
                             float eps, void* stream) {
    if (n_out <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16) {
        if (weight_dtype == DE_BF16)
            return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, out, rows,
                                                                    n_out, width, eps, s);
        return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, weight, out, rows, n_out,
                                                        width, eps, s);
    }
    if (weight_dtype == DE_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, weight, out, rows, n_out,
                                                        width, eps, s);
    return launch_add_rmsnorm<float, float>(resid, delta, weight, out, rows, n_out, width, eps, s);
}

// ------------------------------------------------------------------------------------------
// rotation of q and k by position + write of k and v into the pages of the cache.
//   qkv row = [q heads | k heads | v heads], each head `d` wide.
//   pair (j, j + rot/2) of a head is rotated by angle = float(pos) * inv_freq[j]
//   (half-split pairing, src/layers/rotary_embedding.py:45-54); dims >= rot stay.
//   q is rotated in place; rotated k and v go to
//   pages[(block_table[slot][pos / page] * kv_heads + h) * page + pos % page][:]
//   (position -> page and offset as in src/distengine/paged_kv_cache.py:165-167).
// inv_freq null: no rotation.  write_kv 0: a layer that reads another layer's cache rotates q only.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_slot,
                                     const float* __restrict__ inv_freq, int rot, int heads,
                                     int kv_heads, int d, T* __restrict__ k_pages,
                                     T* __restrict__ v_pages, const int* __restrict__ block_table,
                                     int table_stride, int page, int write_kv, int num_pages,
                                     int* __restrict__ status) {
    const int n = blockIdx.x;
    const int pos = positions[n];
    T* row = qkv + (size_t)n * row_stride;
    const int half = rot / 2;

    size_t kv_base = 0;
    bool can_write = write_kv != 0;
    if (can_write) {
        const int slot = token_slot[n];
        const int page_id = block_table[(size_t)slot * table_stride + pos / page];
        if (page_id < 0 || page_id >= num_pages) {      // a table without a page here: record, skip
            if (threadIdx.x == 0 && threadIdx.y == 0) atomicExch(status, 1);
            can_write = false;
        }
        kv_base = ((size_t)page_id * kv_heads) * page * d + (size_t)(pos % page) * d;
    }
    const size_t head_step = (size_t)page * d;          // from one kv head's slab to the next
    pdl_wait();
    pdl_trigger();

    // rotated pairs: threadIdx.x walks the pair index, threadIdx.y the heads
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float c = 1.0f, s = 0.0f;
        if (inv_freq) {
            const float angle = (float)pos * inv_freq[j];
            c = cosf(angle);
            s = sinf(angle);
        }
        for (int h = threadIdx.y; h < heads + kv_heads; h += blockDim.y) {
            T* x = row + (size_t)h * d;
            const float a = to_float(x[j]), b = to_float(x[j + half]);
            float fa, fb;
            rope_rotate(a, b, c, s, fa, fb);
            const T ra = from_float<T>(fa);
            const T rb = from_float<T>(fb);
            if (h < heads) {
                x[j] = ra;
                x[j + half] = rb;
            } else if (can_write) {
                T* dst = k_pages + kv_base + (size_t)(h - heads) * head_step;
                dst[j] = ra;
                dst[j + half] = rb;
            }
        }
    }
    if (!can_write) return;
    // k dims beyond the rotated width are copied as they are
    for (int j = rot + threadIdx.x; j < d; j += blockDim.x)
        for (int h = threadIdx.y; h < kv_heads; h += blockDim.y)
            k_pages[kv_base + (size_t)h * head_step + j] = row[(size_t)(heads + h) * d + j];
    // v
    for (int j = threadIdx.x; j < d; j += blockDim.x)
        for (int h = threadIdx.y; h < kv_heads; h += blockDim.y)
            v_pages[kv_base + (size_t)h * head_step + j] =
                row[(size_t)(heads + kv_heads + h) * d + j];
}

// The same for bfloat16 rows of 16-byte pieces with every feature rotated (rot == d, d a multiple
// of 16).  A block takes a token: its first threads form the cosines and sines of the token's
// d / 2 angles once, in shared memory, for all heads (that is what the kernel's time went into when
// every thread formed its own: 36 heads repeat the same angles); then a thread takes 8 pairs of one
// head - the pieces j .. j + 7 of both halves - or one piece of a value row, and requests all it
// needs at once.
constexpr int ROPE_MAX_HALF = 128;                           // head sizes up to 256
__global__ void rope_kv_write_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride,
                                            const int* __restrict__ positions,
                                            const int* __restrict__ token_slot,
                                            const float* __restrict__ inv_freq, int heads,
                                            int kv_heads, int d, __nv_bfloat16* __restrict__ k_pages,
                                            __nv_bfloat16* __restrict__ v_pages,
                                            const int* __restrict__ block_table, int table_stride,
                                            int page, int write_kv, int num_pages, int n_tokens,
                                            int* __restrict__ status) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    __shared__ int page_s;
    const int half = d / 2;
    const int per_head = half / 8;                           // rotation items of a head
    const int rotations = (heads + kv_heads) * per_head;
    const int per_token = rotations + kv_heads * (d / 8);    // then the pieces of the value rows
    const int n = blockIdx.x;
    const int pos = positions[n];
    // the angles and the page do not depend on the kernel before this one
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float angle = inv_freq != nullptr ? (float)pos * inv_freq[j] : 0.0f;
        cos_s[j] = cosf(angle);
        sin_s[j] = sinf(angle);
    }
    if (threadIdx.x == blockDim.x - 1) {
        int page_id = -1;
        if (write_kv != 0) {
            page_id = block_table[(size_t)token_slot[n] * table_stride + pos / page];
            if (page_id < 0 || page_id >= num_pages) {  // a table without a page here: record, skip
                atomicExch(status, 1);
                page_id = -1;
            }
        }
        page_s = page_id;
    }
    pdl_wait();
    pdl_trigger();
    __syncthreads();
    const int page_id = page_s;
    __nv_bfloat16* row = qkv + (size_t)n * row_stride;
    for (int local = threadIdx.x; local < per_token; local += blockDim.x) {
        const bool rotation = local < rotations;
        const int h = rotation ? local / per_head : (local - rotations) / (d / 8);
        const int piece = rotation ? local - h * per_head : (local - rotations) - h * (d / 8);
        const int kv_head = rotation ? h - heads : h;
        const size_t kv_offset =
            (((size_t)(page_id < 0 ? 0 : page_id) * kv_heads + (kv_head < 0 ? 0 : kv_head)) * page +
             (size_t)(pos % page)) * d;
        if (!rotation) {
            if (page_id >= 0)
                *reinterpret_cast<uint4*>(v_pages + kv_offset + piece * 8) =
                    *reinterpret_cast<const uint4*>(row + (size_t)(heads + kv_heads + h) * d +
                                                    piece * 8);
            continue;
        }
        __nv_bfloat16* x = row + (size_t)h * d + piece * 8;
        uint4 lo = *reinterpret_cast<const uint4*>(x), hi = *reinterpret_cast<const uint4*>(x + half);
        unsigned* lo_words[4] = {&lo.x, &lo.y, &lo.z, &lo.w};
        unsigned* hi_words[4] = {&hi.x, &hi.y, &hi.z, &hi.w};
#pragma unroll
        for (int e = 0; e < 8; e += 2) {                 // two elements a 32-bit word
            const float a0 = __uint_as_float(*lo_words[e / 2] << 16);
            const float a1 = __uint_as_float(*lo_words[e / 2] & 0xffff0000u);
            const float b0 = __uint_as_float(*hi_words[e / 2] << 16);
            const float b1 = __uint_as_float(*hi_words[e / 2] & 0xffff0000u);
            float fa0, fb0, fa1, fb1;
            rope_rotate(a0, b0, cos_s[piece * 8 + e], sin_s[piece * 8 + e], fa0, fb0);
            rope_rotate(a1, b1, cos_s[piece * 8 + e + 1], sin_s[piece * 8 + e + 1], fa1, fb1);
            const __nv_bfloat162 ra = __floats2bfloat162_rn(fa0, fa1);
            const __nv_bfloat162 rb = __floats2bfloat162_rn(fb0, fb1);
            *lo_words[e / 2] = *reinterpret_cast<const unsigned*>(&ra);
            *hi_words[e / 2] = *reinterpret_cast<const unsigned*>(&rb);
        }
        if (h < heads) {
            *reinterpret_cast<uint4*>(x) = lo;
            *reinterpret_cast<uint4*>(x + half) = hi;
        } else if (page_id >= 0) {
            *reinterpret_cast<uint4*>(k_pages + kv_offset + piece * 8) = lo;
            *reinterpret_cast<uint4*>(k_pages + kv_offset + half + piece * 8) = hi;
        }
    }
}

DE_EXPORT int de_rope_kv_write(int dtype, void* qkv, int row_stride, const int* positions,
                               const int* token_slot, const float* inv_freq, int rot, int heads,
                               int kv_heads, int d, void* k_pages, void* v_pages,
                               const int* block_table, int table_stride, int page, int write_kv,
                               int num_pages, int n, int* status, void* stream) {
    if (n <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16 && d % 16 == 0 && d <= 2 * ROPE_MAX_HALF && (inv_freq == nullptr || rot == d) &&
        row_stride % 8 == 0 &&
        ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0) {
        const int per_token = (heads + kv_heads) * (d / 16) + kv_heads * (d / 8);
        const int threads = per_token >= 256 ? 256 : (per_token + 31) / 32 * 32;
        return de_launch(rope_kv_write_bf16x8_kernel, dim3((unsigned)n), dim3(threads), 0, s, (__nv_bfloat16*)qkv, row_stride, positions, token_slot, inv_freq,
                         heads, kv_heads, d, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                         block_table, table_stride, page, write_kv, num_pages, n, status);
    }
    int tx = 32;
    while (tx < d / 2 && tx < 128) tx <<= 1;
    int ty = 256 / tx;
    dim3 block(tx, ty);
#define LAUNCH(T)                                                                              \
    return de_launch(rope_kv_write_kernel<T>, dim3(n), block, 0, s, (T*)qkv, row_stride,       \
                     positions, token_slot, inv_freq, rot, heads, kv_heads, d, (T*)k_pages,    \
                     (T*)v_pages, block_table, table_stride, page, write_kv, num_pages, status)
    if (dtype == DE_BF16) LAUNCH(__nv_bfloat16);
    LAUNCH(float);
#undef LAUNCH
}

// ------------------------------------------------------------------------------------------
// out[n, i] = T( silu(gate) * up ), gate = x[n, i], up = x[n, inner + i]; silu(z) = z * sigmoid(z)
// (src/layers/activation.py:6-9; the packed [gate | up] row as in src/models/llama.py:26).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inner,
                                size_t total) {
    pdl_wait();
    pdl_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / inner;
        const int i = (int)(idx - n * inner);
        const float g = to_float(x[n * 2 * inner + i]);
        const float u = to_float(x[n * 2 * inner + inner + i]);
        const float sg = g / (1.0f + expf(-g));
        out[idx] = from_float<T>(sg * u);
    }
}

// inner a multiple of 4: four outputs a thread, 8- or 16-byte accesses
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int inner,
                                    size_t total_quads) {
    pdl_wait();
    pdl_trigger();
    const int quads = inner >> 2;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_quads;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / quads;
        const int i = 4 * (int)(idx - n * quads);
        float g[4], u[4], y[4];
        Vec4<T>::load(x + n * 2 * inner + i, g);
        Vec4<T>::load(x + n * 2 * inner + inner + i, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
        Vec4<T>::store(out + n * inner + i, y);
    }
}

DE_EXPORT int de_silu_mul(int dtype, const void* x, void* out, int n, int inner, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const bool vec = inner % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const size_t total = vec ? (size_t)n * (inner / 4) : (size_t)n * inner;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == DE_BF16) {
        if (vec)
            return de_launch(silu_mul_vec_kernel<__nv_bfloat16>, dim3((unsigned)blocks),
                             dim3(threads), 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                             inner, total);
        return de_launch(silu_mul_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0,
                         s, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, inner, total);
    }
    if (vec)
        return de_launch(silu_mul_vec_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, s,
                         (const float*)x, (float*)out, inner, total);
    return de_launch(silu_mul_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, s,
                     (const float*)x, (float*)out, inner, total);
}

// ------------------------------------------------------------------------------------------
// sampling over rows of float32 logits.
//   temperature 0: arg-max, the lowest id wins a tie (src/layers/sampler.py:8).
//   temperature > 0: a draw from softmax(logits / T) by the Gumbel-max rule,
//     arg-max_i( logits_i / T - log(-log(u_i)) ),  u_i a counter-based uniform of
//     (seed, position, i): the draw depends on the request's own seed and position only, never on
//     the batch.  The reference samples greedily only.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float uniform_of(unsigned long long base, int i) {
    unsigned long long z = base + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return ((float)(z >> 41) + 0.5f) * (1.0f / 8388608.0f);     // 23 bits + 0.5: exact, in (0,1)
}

__global__ void __launch_bounds__(1024)
sample_rows_kernel(const float* __restrict__ logits, int vocab,
                                   const float* __restrict__ temperature,
                                   const long long* __restrict__ seed,
                                   const int* __restrict__ position, int* __restrict__ out) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float t = temperature ? temperature[r] : 0.0f;
    unsigned long long base = 0;
    if (t > 0.0f)
        base = (unsigned long long)seed[r] * 0x9E3779B97F4A7C15ull +
               (unsigned long long)(long long)position[r] * 0xD1B54A32D192ED03ull;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (t > 0.0f) v = v / t - logf(-logf(uniform_of(base, i)));
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    };
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        // 16-byte loads, eight of them requested before the first is looked at
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int quads = vocab >> 2;
        for (int q0 = threadIdx.x; q0 < quads; q0 += 8 * blockDim.x) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int q = q0 + u * blockDim.x;
                v[u] = q < quads ? row4[q] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int q = q0 + u * blockDim.x;
                if (q < quads) {
                    take(v[u].x, 4 * q); take(v[u].y, 4 * q + 1);
                    take(v[u].z, 4 * q + 2); take(v[u].w, 4 * q + 3);
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) take(row[i], i);
    }
    // reduce (value, lowest index on ties) over the block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
            bv = ov; bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        bv = lane < warps ? best_v[lane] : -INFINITY;
        bi = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
                bv = ov; bi = oi;
            }
        }
        if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
    }
}

DE_EXPORT int de_sample_rows(const float* logits, int rows, int vocab, const float* temperature,
                             const long long* seed, const int* position, int* out, void* stream) {
    if (rows <= 0) return 0;
    return de_launch(sample_rows_kernel, dim3(rows), dim3(1024), 0, (cudaStream_t)stream, logits,
                     vocab, temperature, seed, position, out);
}
