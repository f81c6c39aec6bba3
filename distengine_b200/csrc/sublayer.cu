// Row kernels for blocks whose norm stands on a sublayer's output instead of its input, with a
// gate on that output, and for a stream that is a weighted average over the depth:
//
//   norm_stream        x <- x / sqrt(mean(x^2) + eps) * w in place on the float32 stream (the norm
//                      of the embedding rows), with a copy in the activation type
//   gated_normed_add   g = y * sigmoid(z + b);  out = x + g / sqrt(mean(g^2) + eps) * w
//                      y a sublayer's result, z the gate's product on the sublayer's input
//   depth_mix          x = sum over j < count of c[j] * X_j    (X_j the embedding rows and every
//                      layer's result so far, c a learned vector of the layer)
//   poly_norm          out = a N(z) + b N(z^2) + c N(z^3) + e, N dividing a row by its root mean
//                      square (eps inside the root), powers element by element
//
// All sums, statistics and the stream are float32 whatever the activation type; every kernel that
// writes the stream can also write its rounding to the activation type, which the next matrix
// products read.  One block a row (depth_mix: a thread four elements); a row's sums have an order
// that depends on the block's size only.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T, typename W>
__global__ void norm_stream_kernel(float* __restrict__ x, const W* __restrict__ weight,
                                   T* __restrict__ rows, int width, float eps) {
    __shared__ float scratch[33];
    const size_t row = blockIdx.x;
    float* xr = x + row * width;
    pdl_wait();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    pdl_trigger();
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] * inv * to_float(weight[i]);
        xr[i] = v;
        if (rows != nullptr) rows[row * width + i] = from_float<T>(v);
    }
}

// Y: the sublayer's result (activation type or float32); T: the activation type of the gate's
// product and of the rounded copy.  `in` and `out` may be the same rows or different ones.
template <typename T, typename Y, typename W>
__global__ void gated_normed_add_kernel(const Y* __restrict__ y, const T* __restrict__ gate,
                                        int ld_gate, const float* __restrict__ bias,
                                        const W* __restrict__ weight, const float* in,
                                        float* out, T* __restrict__ rows, int width, float eps) {
    extern __shared__ float g[];                     // [width]
    __shared__ float scratch[33];
    const size_t row = blockIdx.x;
    pdl_wait();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_float(y[row * width + i]) *
                        sigmoid_f(to_float(gate[row * ld_gate + i]) + bias[i]);
        g[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    pdl_trigger();
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = in[row * width + i] + g[i] * inv * to_float(weight[i]);
        out[row * width + i] = v;
        if (rows != nullptr) rows[row * width + i] = from_float<T>(v);
    }
}

// history [count][total] float32 with `stride` elements between two members.
template <typename T>
__global__ void depth_mix_kernel(const float* __restrict__ history, size_t stride,
                                 const float* __restrict__ coef, int count, size_t total,
                                 float* __restrict__ x, T* __restrict__ rows) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int j = 0; j < count; ++j) s = fmaf(coef[j], history[j * stride + i], s);
        x[i] = s;
        if (rows != nullptr) rows[i] = from_float<T>(s);
    }
}

// 16 bytes of T as floats and back
template <typename T> struct Chunk;
template <> struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* f) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* f) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Three sums over a block at once; every thread gets the results.  The order of the additions
// depends on the block's size only.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float* scratch /* 99 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    c = warp_sum(c);
    if (lane == 0) {
        scratch[warp] = a;
        scratch[32 + warp] = b;
        scratch[64 + warp] = c;
    }
    __syncthreads();
    if (warp < 3) {
        float t = lane < warps ? scratch[32 * warp + lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[96 + warp] = t;
    }
    __syncthreads();
    a = scratch[96];
    b = scratch[97];
    c = scratch[98];
}

// VEC: rows are whole 16-byte pieces at 16-byte addresses; a thread then takes pieces, and the
// second pass finds the row in the caches.
template <typename T, bool VEC>
__global__ void poly_norm_kernel(const T* __restrict__ z, int ldz, const float* __restrict__ coef,
                                 T* __restrict__ out, int ldo, int cols, float eps) {
    __shared__ float scratch[99];
    constexpr int PN = Chunk<T>::N;
    const size_t row = blockIdx.x;
    const T* zr = z + row * ldz;
    pdl_wait();
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    if (VEC) {
        for (int i = threadIdx.x * PN; i < cols; i += blockDim.x * PN) {
            float f[PN];
            Chunk<T>::load(zr + i, f);
#pragma unroll
            for (int e = 0; e < PN; ++e) {
                const float v = f[e], v2 = v * v, v3 = v2 * v;
                s1 = fmaf(v, v, s1);
                s2 = fmaf(v2, v2, s2);
                s3 = fmaf(v3, v3, s3);
            }
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = to_float(zr[i]), v2 = v * v, v3 = v2 * v;
            s1 = fmaf(v, v, s1);
            s2 = fmaf(v2, v2, s2);
            s3 = fmaf(v3, v3, s3);
        }
    }
    block_sum3(s1, s2, s3, scratch);
    const float n = (float)cols;
    const float i1 = coef[0] / sqrtf(s1 / n + eps);
    const float i2 = coef[1] / sqrtf(s2 / n + eps);
    const float i3 = coef[2] / sqrtf(s3 / n + eps);
    const float e0 = coef[3];
    pdl_trigger();
    if (VEC) {
        for (int i = threadIdx.x * PN; i < cols; i += blockDim.x * PN) {
            float f[PN];
            Chunk<T>::load(zr + i, f);
#pragma unroll
            for (int e = 0; e < PN; ++e) {
                const float v = f[e], v2 = v * v;
                f[e] = v * i1 + v2 * i2 + v2 * v * i3 + e0;
            }
            Chunk<T>::store(out + row * ldo + i, f);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = to_float(zr[i]), v2 = v * v;
            out[row * ldo + i] = from_float<T>(v * i1 + v2 * i2 + v2 * v * i3 + e0);
        }
    }
}

int row_threads(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

}  // namespace

DE_EXPORT int de_norm_stream(int dtype, int weight_dtype, float* x, const void* weight, void* rows,
                             int n, int width, float eps, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = row_threads(width);
#define NS(T, W)                                                                                 \
    return de_launch(norm_stream_kernel<T, W>, dim3(n), dim3(threads), 0, s, x, (const W*)weight, \
                     (T*)rows, width, eps)
    if (dtype == DE_BF16) {
        if (weight_dtype == DE_BF16) NS(__nv_bfloat16, __nv_bfloat16);
        NS(__nv_bfloat16, float);
    }
    if (weight_dtype == DE_BF16) NS(float, __nv_bfloat16);
    NS(float, float);
#undef NS
}

// dtype: of gate and rows; y_dtype: of y.
DE_EXPORT int de_gated_normed_add(int dtype, int y_dtype, int weight_dtype, const void* y,
                                  const void* gate, int ld_gate, const float* bias,
                                  const void* weight, const float* in, float* out, void* rows,
                                  int n, int width, float eps, void* stream) {
    if (n <= 0) return 0;
    if (dtype == DE_F32 && y_dtype != DE_F32) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = row_threads(width);
    const size_t smem = (size_t)width * sizeof(float);
#define GNA(T, Y, W)                                                                             \
    do {                                                                                         \
        if (smem > 48 * 1024) {                                                                  \
            cudaError_t e = cudaFuncSetAttribute(gated_normed_add_kernel<T, Y, W>,               \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                                 (int)smem);                                     \
            if (e != cudaSuccess) return (int)e;                                                 \
        }                                                                                        \
        return de_launch(gated_normed_add_kernel<T, Y, W>, dim3(n), dim3(threads), smem, s,      \
                         (const Y*)y, (const T*)gate, ld_gate, bias, (const W*)weight, in, out,  \
                         (T*)rows, width, eps);                                                  \
    } while (0)
    if (dtype == DE_BF16) {
        if (y_dtype == DE_BF16) {
            if (weight_dtype == DE_BF16) GNA(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
            GNA(__nv_bfloat16, __nv_bfloat16, float);
        }
        if (weight_dtype == DE_BF16) GNA(__nv_bfloat16, float, __nv_bfloat16);
        GNA(__nv_bfloat16, float, float);
    }
    if (weight_dtype == DE_BF16) GNA(float, float, __nv_bfloat16);
    GNA(float, float, float);
#undef GNA
}

DE_EXPORT int de_depth_mix(int dtype, const float* history, long long stride, const float* coef,
                           int count, long long total, float* x, void* rows, void* stream) {
    if (total <= 0 || count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    size_t blocks = ((size_t)total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == DE_BF16)
        return de_launch(depth_mix_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s,
                         history, (size_t)stride, coef, count, (size_t)total, x,
                         (__nv_bfloat16*)rows);
    return de_launch(depth_mix_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, history,
                     (size_t)stride, coef, count, (size_t)total, x, (float*)rows);
}

DE_EXPORT int de_poly_norm(int dtype, const void* z, int ldz, const float* coef, void* out,
                           int ldo, int n, int cols, float eps, void* stream) {
    if (n <= 0 || cols <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = row_threads(cols);
    const int pn = dtype == DE_BF16 ? 8 : 4;
    const bool vec = cols % pn == 0 && ldz % pn == 0 && ldo % pn == 0 &&
                     (uintptr_t)z % 16 == 0 && (uintptr_t)out % 16 == 0;
#define POLY(T, V)                                                                             \
    return de_launch(poly_norm_kernel<T, V>, dim3(n), dim3(threads), 0, s, (const T*)z, ldz,   \
                     coef, (T*)out, ldo, cols, eps)
    if (dtype == DE_BF16) {
        if (vec) POLY(__nv_bfloat16, true);
        POLY(__nv_bfloat16, false);
    }
    if (vec) POLY(float, true);
    POLY(float, false);
#undef POLY
}
