// Kernels of latent attention: keys and values of all heads are read from one small latent per
// token, which is what the pages hold, [c (rank) | rotated key part (rot)] a token.
//
//   latent_write   c = rms_norm(first `rank` columns) * weight and the rotated key part into the
//                  pages; every head's rotated query part into the rows that the attention reads
//   heads_product  one small product per head: out[n, h, :] = W[h] a[n, h, :]
//
// With the per-head key matrix folded into the query (q' = W_uk[h]^T q, the score of a key is
// q' . c + q_rot . k_rot) and the per-head value matrix applied after the weighted sum over c,
// attention over the latent is attention with one key/value head whose values are the first
// `rank` features of its keys.
//
// Angles are formed in double precision from the position and the frequency (a product in 32-bit
// loses digits at far positions); cosine and sine are multiplied by `magnitude`.  Norm statistics,
// sums of products and the gate are float32.

#include "rows_product.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

// One block a token.  kv row = [c raw (rank) | key part (rot)], q row = H heads of [plain (dim) |
// rotated part (rot)]; qa row = H heads of [.. (rank, written by heads_product) | rotated (rot)].
template <typename T, typename W>
__global__ void latent_write_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ kv,
                                    int ldkv, T* __restrict__ qa, int ldqa,
                                    const int* __restrict__ positions,
                                    const int* __restrict__ token_slot,
                                    const double* __restrict__ freq, float magnitude,
                                    const W* __restrict__ norm_w, float eps, int H, int dim,
                                    int rot, int rank, T* __restrict__ pages,
                                    const int* __restrict__ block_table, int table_stride,
                                    int page, int num_pages, int* __restrict__ status) {
    extern __shared__ float cs[];                    // [rot]: cosines, then sines, of the position
    __shared__ float scratch[33];
    const int n = blockIdx.x;
    const int pos = positions[n], slot = token_slot[n];
    const int half = rot / 2, row_dim = rank + rot;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)pos * freq[i], &s, &c);
        cs[i] = (float)c * magnitude;
        cs[half + i] = (float)s * magnitude;
    }
    pdl_wait();
    const int page_id = block_table[(size_t)slot * table_stride + pos / page];
    const T* kvr = kv + (size_t)n * ldkv;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(kvr[i]);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);   // also a barrier
    pdl_trigger();
    // the queries' rotated parts
    const T* qr = q + (size_t)n * ldq;
    T* qar = qa + (size_t)n * ldqa;
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float a = to_float(qr[h * (dim + rot) + dim + i]);
        const float b = to_float(qr[h * (dim + rot) + dim + half + i]);
        float ra, rb;
        rope_rotate(a, b, cs[i], cs[half + i], ra, rb);
        qar[h * row_dim + rank + i] = from_float<T>(ra);
        qar[h * row_dim + rank + half + i] = from_float<T>(rb);
    }
    if (page_id < 0 || page_id >= num_pages) {       // never written outside the pool
        if (threadIdx.x == 0) atomicExch(status, 1);
        return;
    }
    T* dst = pages + ((size_t)page_id * page + (size_t)(pos % page)) * row_dim;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(from_float<T>(to_float(kvr[i]) * inv));
        dst[i] = from_float<T>(v * to_float(norm_w[i]));
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float ra, rb;
        rope_rotate(to_float(kvr[rank + i]), to_float(kvr[rank + half + i]), cs[i], cs[half + i],
                    ra, rb);
        dst[rank + i] = from_float<T>(ra);
        dst[rank + half + i] = from_float<T>(rb);
    }
}

// out[n, h * ldo_h + j] = sum_i a[n, h * lda_h + i] * w[h][j][i] for j < cols, i < depth, times
// sigmoid(gate[n, h * cols + j]) where a gate is given.  grid (row tiles, column tiles, heads).
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(rows_product::THREADS)
heads_product_kernel(const TA* __restrict__ a, int lda, int lda_h, const TW* __restrict__ w,
                     TO* __restrict__ out, int ldo, int ldo_h, const TW* __restrict__ gate,
                     int ld_gate, int n, int cols, int depth, int vec_a, int vec_w) {
    __shared__ __align__(16) float smem[rows_product::SMEM_FLOATS];
    const int r0 = blockIdx.x * rows_product::TILE, c0 = blockIdx.y * rows_product::TILE;
    const int h = blockIdx.z;
    const TW* wt = w + ((size_t)h * cols + c0) * depth;
    float acc[4][4];
    pdl_wait();
    rows_product::tile<TA, TW>(
        [&](int r) -> const TA* {
            return r0 + r < n ? a + (size_t)(r0 + r) * lda + (size_t)h * lda_h : nullptr;
        },
        wt, depth, min(rows_product::TILE, cols - c0), depth, vec_a != 0, vec_w != 0, smem, acc);
    pdl_trigger();
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + tr * 4 + i;
        if (r >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tc * 4 + j;
            if (c >= cols) continue;
            float y = acc[i][j];
            if (gate != nullptr) {
                const float g = to_float(gate[(size_t)r * ld_gate + (size_t)h * cols + c]);
                y = y / (1.0f + expf(-g));
            }
            out[(size_t)r * ldo + (size_t)h * ldo_h + c] = from_float<TO>(y);
        }
    }
}

}  // namespace

DE_EXPORT int de_latent_write(int dtype, int weight_dtype, const void* q, int ldq, const void* kv,
                              int ldkv, void* qa, int ldqa, const int* positions,
                              const int* token_slot, const double* freq, float magnitude,
                              const void* norm_w, float eps, int H, int dim, int rot, int rank,
                              void* pages, const int* block_table, int table_stride, int page,
                              int num_pages, int n, int* status, void* stream) {
    if (n <= 0) return 0;
    if (rot < 0 || rot % 2 || rank <= 0 || dim <= 0 || H <= 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
#define LW(T, W)                                                                                \
    return de_launch(latent_write_kernel<T, W>, dim3(n), dim3(128), smem, s, (const T*)q, ldq,   \
                     (const T*)kv, ldkv, (T*)qa, ldqa, positions, token_slot, freq, magnitude,  \
                     (const W*)norm_w, eps, H, dim, rot, rank, (T*)pages, block_table,          \
                     table_stride, page, num_pages, status)
    if (dtype == DE_BF16) {
        if (weight_dtype == DE_BF16) LW(__nv_bfloat16, __nv_bfloat16);
        LW(__nv_bfloat16, float);
    }
    if (weight_dtype == DE_BF16) LW(float, __nv_bfloat16);
    LW(float, float);
#undef LW
}

// a_dtype / w_dtype / out_dtype: DE_F32 or DE_BF16; the gate (optional) has the weights' type.
DE_EXPORT int de_heads_product(int a_dtype, int w_dtype, int out_dtype, const void* a, int lda,
                               int lda_h, const void* w, void* out, int ldo, int ldo_h,
                               const void* gate, int ld_gate, int n, int heads, int cols,
                               int depth, void* stream) {
    if (n <= 0 || heads <= 0 || cols <= 0) return 0;
    if (depth <= 0 || heads > 65535) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((n + rows_product::TILE - 1) / rows_product::TILE,
                    (cols + rows_product::TILE - 1) / rows_product::TILE, heads);
    if (grid.y > 65535) return -2;
    const int asz = a_dtype == DE_BF16 ? 2 : 4, wsz = w_dtype == DE_BF16 ? 2 : 4;
    const int vec_a = ((uintptr_t)a % (4 * asz) == 0) && (lda % 4 == 0) && (lda_h % 4 == 0);
    const int vec_w = ((uintptr_t)w % (4 * wsz) == 0) && (depth % 4 == 0);
#define HP(TA, TW, TO)                                                                          \
    return de_launch(heads_product_kernel<TA, TW, TO>, grid, dim3(rows_product::THREADS), 0, s, \
                     (const TA*)a, lda, lda_h, (const TW*)w, (TO*)out, ldo, ldo_h,              \
                     (const TW*)gate, ld_gate, n, cols, depth, vec_a, vec_w)
    if (w_dtype == DE_BF16) {
        if (a_dtype == DE_BF16 && out_dtype == DE_BF16) HP(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
        if (a_dtype == DE_F32 && out_dtype == DE_BF16) HP(float, __nv_bfloat16, __nv_bfloat16);
        if (a_dtype == DE_BF16 && out_dtype == DE_F32) HP(__nv_bfloat16, __nv_bfloat16, float);
        return -2;
    }
    if (a_dtype == DE_F32 && out_dtype == DE_F32) HP(float, float, float);
    return -2;
#undef HP
}
