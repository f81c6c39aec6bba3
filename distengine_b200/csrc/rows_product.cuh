// A tile of a matrix product whose rows are found through a function: C[r, j] = sum_i A(r)[i] *
// W[j][i] for a tile of 64 rows and 64 columns, on the CUDA cores with float32 sums.  Every output
// is one chain of multiply-adds over i in ascending order, so a row's result does not depend on
// which rows share its tile, its step or its batch.  The kernels that gather rows (one product per
// head, one product per expert) are built on it.
//
// 256 threads; thread (tr, tc) = (tid / 16, tid % 16) holds rows 4 tr .. 4 tr + 3 and columns
// 4 tc .. 4 tc + 3 of the tile.  Operands pass shared memory in slices of 16 along i, stored with i
// outermost so that a thread reads its four rows and its four columns as one float4 each.
#pragma once

#include "common.cuh"

namespace rows_product {

constexpr int TILE = 64;        // rows and columns of a tile
constexpr int SLICE = 16;       // of i, a stage
constexpr int PITCH = TILE + 4;
constexpr int THREADS = 256;
constexpr int SMEM_FLOATS = 2 * SLICE * PITCH;

// Four consecutive elements from `p` (null: zeros) starting at i, zeros from `depth` on.
template <typename T>
__device__ __forceinline__ void load4(const T* p, int i, int depth, bool vec, float (&v)[4]) {
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = 0.0f;
    if (p == nullptr || i >= depth) return;
    if (vec && i + 4 <= depth) {
        if constexpr (sizeof(T) == 4) {
            const float4 t = *reinterpret_cast<const float4*>(p + i);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
            const uint2 t = *reinterpret_cast<const uint2*>(p + i);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
            v[0] = __low2float(a); v[1] = __high2float(a);
            v[2] = __low2float(b); v[3] = __high2float(b);
        }
        return;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
        if (i + u < depth) v[u] = to_float(p[i + u]);
}

// `a_row(r)`: row r of the tile (0 .. 63) as a pointer to its `depth` elements, or null for a row
// that does not exist.  `w`: the first of the tile's columns, rows of W `ldw` apart; `cols`: how
// many of the 64 columns exist.  `vec_a` / `vec_w`: every row of A / W starts on a 16-byte (float)
// or 8-byte (bfloat16) boundary, so four elements may come in one load.
template <typename TA, typename TW, typename RowA>
__device__ __forceinline__ void tile(RowA a_row, const TW* __restrict__ w, int ldw, int cols,
                                     int depth, bool vec_a, bool vec_w, float* smem,
                                     float (&acc)[4][4]) {
    float* As = smem;                         // [SLICE][PITCH]
    float* Ws = smem + SLICE * PITCH;
    const int tid = threadIdx.x;
    const int tr = tid >> 4, tc = tid & 15;
    const int lr = tid >> 2, lk = (tid & 3) * 4;          // what this thread fetches: row, i
    const TA* arow = a_row(lr);
    const TW* wrow = lr < cols ? w + (size_t)lr * ldw : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < depth; k0 += SLICE) {
        float av[4], wv[4];
        load4<TA>(arow, k0 + lk, depth, vec_a, av);
        load4<TW>(wrow, k0 + lk, depth, vec_w, wv);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            As[(lk + u) * PITCH + lr] = av[u];
            Ws[(lk + u) * PITCH + lr] = wv[u];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SLICE; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(As + k * PITCH + tr * 4);
            const float4 b = *reinterpret_cast<const float4*>(Ws + k * PITCH + tc * 4);
            const float ar[4] = {a.x, a.y, a.z, a.w}, bc[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], bc[j], acc[i][j]);
        }
    }
}

template <typename T>
__host__ __device__ __forceinline__ bool rows_aligned(const void* base, long long ld) {
    const unsigned long long step = sizeof(T) == 4 ? 16 : 8;
    return ((unsigned long long)base % step) == 0 && ((unsigned long long)ld * sizeof(T)) % step == 0;
}

}  // namespace rows_product
