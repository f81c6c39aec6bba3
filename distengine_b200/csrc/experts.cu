// Routed experts: every token goes through the `top` experts whose router logits are largest, and
// their outputs are summed with the softmax over the chosen logits alone.
//
//   route    z = W_r h + b in float32, the `top` largest (ties: the lower index), softmax over them
//   group    the (token, choice) pairs sorted by expert into segments that start at multiples of
//            64 slots, so that a tile of 64 slots belongs to one expert
//   up       inner[slot] = act(W_up[e] h[token])            one tile of rows_product a block
//   down     y[pair] = W_down[e] inner[slot]
//   combine  out[n] = sum_k weight[n, k] * y[n * top + k]   float32, in the order of the choices
//
// A second way to score (`mode` 1): s = softmax(z) over all router outputs, the choice goes by
// s + bias (a correction that does not enter the weights), the weights are the chosen s as they
// are.  The router may have more outputs than there are experts: the outputs from `experts` on
// stand for experts that hand their input on (the grouping leaves their pairs out, `combine` adds
// weight * h for them).  An expert's up product may have no activation (kind 5), for experts whose
// gate and up rows are stacked and joined by a kernel after the product.
//
// Every output element is one chain of multiply-adds over its inputs in ascending order, and a
// token's result does not depend on which tokens share its tile, its expert or its step.  The
// number of tiles that are launched depends on the number of tokens only (tiles without an expert
// return at once), so a step's launches can be replayed from a CUDA graph.

#include "rows_product.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int SEG = rows_product::TILE;     // segments of an expert start at multiples of this
constexpr int MAX_TOP = 32;

// One block of eight warps a token.  Warp w takes the w-th eighth of the features for all experts
// (eight experts at a time, eight chains of multiply-adds side by side); a logit is the sum of the
// warps' shares in the order of the warps, plus the bias.  The order of the sums is fixed, so a
// token's logits do not depend on its step.  Then warp 0 picks the `top` largest (ties: the lower
// index) and forms the softmax over them.  Shared memory: [9][experts] floats.
constexpr int ROUTE_WARPS = 8;
template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ w,
             const float* __restrict__ bias, int n, int width, int experts, int top, int mode,
             int* __restrict__ chosen, float* __restrict__ weight) {
    extern __shared__ float zs[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    float* z = zs + (size_t)ROUTE_WARPS * experts;
    pdl_wait();
    pdl_trigger();
    const T* x = h + (size_t)row * ldh;
    const int slice = ((width + ROUTE_WARPS - 1) / ROUTE_WARPS + 31) / 32 * 32;
    const int i0 = warp * slice, i1 = min(width, i0 + slice);
    for (int e0 = 0; e0 < experts; e0 += 8) {
        float s[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) s[u] = 0.0f;
        const float* wr = w + (size_t)e0 * width;
        if (e0 + 8 <= experts) {
#pragma unroll 2
            for (int i = i0 + lane; i < i1; i += 32) {
                const float xv = to_float(x[i]);
#pragma unroll
                for (int u = 0; u < 8; ++u) s[u] = fmaf(xv, wr[(size_t)u * width + i], s[u]);
            }
        } else {
            for (int i = i0 + lane; i < i1; i += 32) {
                const float xv = to_float(x[i]);
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (e0 + u < experts) s[u] = fmaf(xv, wr[(size_t)u * width + i], s[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float t = warp_sum(s[u]);
            if (lane == 0 && e0 + u < experts) zs[(size_t)warp * experts + e0 + u] = t;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += ROUTE_WARPS * 32) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < ROUTE_WARPS; ++k) t += zs[(size_t)k * experts + e];
        z[e] = mode == 1 ? t : t + bias[e];
    }
    __syncthreads();
    if (warp != 0) return;
    float best[MAX_TOP];
    float total = 0.0f;
    if (mode == 1) {
        // scores over all outputs; z becomes score + correction, the scores stay in zs
        float top_z = -INFINITY;
        for (int e = lane; e < experts; e += 32) top_z = fmaxf(top_z, z[e]);
        top_z = warp_max(top_z);
        float sum = 0.0f;
        for (int e = lane; e < experts; e += 32) sum += expf(z[e] - top_z);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) {
            const float sc = expf(z[e] - top_z) / sum;
            zs[e] = sc;
            z[e] = sc + bias[e];
        }
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float v = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float c = z[e];
            if (c > v || (c == v && e < at)) { v = c; at = e; }
        }
        if (at == 0x7fffffff) v = -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > v || (ov == v && oa < at)) { v = ov; at = oa; }
        }
        best[k] = v;
        if (lane == 0) {
            chosen[(size_t)row * top + k] = at;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (mode == 1) {
        if (lane == 0)
            for (int k = 0; k < top; ++k)
                weight[(size_t)row * top + k] = zs[chosen[(size_t)row * top + k]];
        return;
    }
    for (int k = 0; k < top; ++k) total += expf(best[k] - best[0]);
    if (lane == 0)
        for (int k = 0; k < top; ++k)
            weight[(size_t)row * top + k] = expf(best[k] - best[0]) / total;
}

// One block.  pair_of [slots] (slots = tiles * SEG), tile_expert [tiles], slot_of [pairs].
// `seg`: the slots of a tile (a segment of an expert starts at a multiple of it).
__global__ void group_kernel(const int* __restrict__ chosen, int pairs, int experts, int tiles,
                             int seg, int* __restrict__ pair_of, int* __restrict__ tile_expert,
                             int* __restrict__ slot_of) {
    extern __shared__ int sh[];                      // [experts] counts, then [experts] cursors
    int* count = sh;
    int* cursor = sh + experts;
    pdl_wait();                 // the lists may still be read by the layer before
    pdl_trigger();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int t = threadIdx.x; t < tiles; t += blockDim.x) tile_expert[t] = -1;
    for (int i = threadIdx.x; i < tiles * seg; i += blockDim.x) pair_of[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            cursor[e] = at;
            const int t = (count[e] + seg - 1) / seg;
            for (int i = 0; i < t; ++i) tile_expert[at / seg + i] = e;
            at += t * seg;
        }
    }
    __syncthreads();
    // which slot of its expert's segment a pair takes does not matter to its result
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= experts) { slot_of[p] = -1; continue; }
        const int slot = atomicAdd(&cursor[e], 1);
        pair_of[slot] = p;
        slot_of[p] = slot;
    }
}

// inner[slot, j] = act(sum_i h[token(slot), i] * up[e][j][i]); grid (tiles, column tiles of ff).
template <typename T>
__global__ void __launch_bounds__(rows_product::THREADS)
expert_up_kernel(const T* __restrict__ h, int ldh, const T* __restrict__ up,
                 const int* __restrict__ pair_of, const int* __restrict__ tile_expert, int top,
                 int width, int ff, T* __restrict__ inner, int act, int vec_a, int vec_w) {
    __shared__ __align__(16) float smem[rows_product::SMEM_FLOATS];
    __shared__ int pair_s[SEG];
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int s0 = blockIdx.x * SEG, c0 = blockIdx.y * rows_product::TILE;
    if (threadIdx.x < SEG) pair_s[threadIdx.x] = pair_of[s0 + threadIdx.x];
    __syncthreads();
    float acc[4][4];
    rows_product::tile<T, T>(
        [&](int r) -> const T* {
            const int p = pair_s[r];
            return p >= 0 ? h + (size_t)(p / top) * ldh : nullptr;
        },
        up + ((size_t)e * ff + c0) * width, width, min(rows_product::TILE, ff - c0), width,
        vec_a != 0, vec_w != 0, smem, acc);
    pdl_trigger();
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = tr * 4 + i;
        if (pair_s[r] < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tc * 4 + j;
            if (c < ff) inner[(size_t)(s0 + r) * ff + c] =
                from_float<T>(act == 5 ? acc[i][j] : de_activate(acc[i][j], act));
        }
    }
}

// y[pair, j] = sum_i inner[slot, i] * down[e][j][i]; grid (tiles, column tiles of width).
template <typename T>
__global__ void __launch_bounds__(rows_product::THREADS)
expert_down_kernel(const T* __restrict__ inner, const T* __restrict__ down,
                   const int* __restrict__ pair_of, const int* __restrict__ tile_expert,
                   int width, int ff, T* __restrict__ y, int vec_a, int vec_w) {
    __shared__ __align__(16) float smem[rows_product::SMEM_FLOATS];
    __shared__ int pair_s[SEG];
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int s0 = blockIdx.x * SEG, c0 = blockIdx.y * rows_product::TILE;
    if (threadIdx.x < SEG) pair_s[threadIdx.x] = pair_of[s0 + threadIdx.x];
    __syncthreads();
    float acc[4][4];
    rows_product::tile<T, T>(
        [&](int r) -> const T* {
            return pair_s[r] >= 0 ? inner + (size_t)(s0 + r) * ff : nullptr;
        },
        down + ((size_t)e * width + c0) * ff, ff, min(rows_product::TILE, width - c0), ff,
        vec_a != 0, vec_w != 0, smem, acc);
    pdl_trigger();
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = pair_s[tr * 4 + i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + tc * 4 + j;
            if (c < width) y[(size_t)p * width + c] = from_float<T>(acc[i][j]);
        }
    }
}

// One block a slot.
template <typename T>
__global__ void gather_kernel(const T* __restrict__ h, int ldh, const int* __restrict__ pair_of,
                              int top, int width, T* __restrict__ rows) {
    pdl_wait();
    pdl_trigger();
    const int pair = pair_of[blockIdx.x];
    T* dst = rows + (size_t)blockIdx.x * width;
    const T* src = pair >= 0 ? h + (size_t)(pair / top) * ldh : nullptr;
    constexpr int PER = 16 / sizeof(T);
    const bool vec = width % PER == 0 && ((uintptr_t)rows % 16) == 0 &&
                     (src == nullptr || ((uintptr_t)src % 16) == 0);
    if (vec) {
        for (int i = threadIdx.x; i < width / PER; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] =
                src ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            dst[i] = src ? src[i] : from_float<T>(0.0f);
    }
}

// chosen / experts / h: a pair whose choice is not below `experts` adds weight * h[n] (an expert
// that hands its input on); chosen null: every pair has a row of y.
template <typename T>
__global__ void combine_kernel(const T* __restrict__ y, const float* __restrict__ weight, int top,
                               int width, size_t total, float* __restrict__ out,
                               const int* __restrict__ chosen, int experts,
                               const T* __restrict__ h, int ldh) {
    pdl_wait();
    pdl_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / width;
        const int i = (int)(idx - n * width);
        float s = 0.0f;
        for (int k = 0; k < top; ++k) {
            const bool hands_on = chosen != nullptr && chosen[n * top + k] >= experts;
            const float v = hands_on ? to_float(h[n * ldh + i])
                                     : to_float(y[(n * top + k) * width + i]);
            s = fmaf(weight[n * top + k], v, s);
        }
        out[idx] = s;
    }
}

}  // namespace

// How many tiles (of `seg` slots) the grouped pairs of n tokens can take at most.
DE_EXPORT int de_experts_tiles(int n, int top, int experts, int seg) {
    const long long pairs = (long long)n * top;
    const long long most = pairs / seg + (experts < pairs ? experts : pairs);
    return (int)(most < 1 ? 1 : most);
}

DE_EXPORT int de_experts_route(int dtype, const void* h, int ldh, const float* w,
                               const float* bias, int n, int width, int experts, int top,
                               int mode, int* chosen, float* weight, void* stream) {
    if (n <= 0) return 0;
    if (top <= 0 || top > MAX_TOP || top > experts || experts > 1024) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = ROUTE_WARPS;
    const size_t smem = (size_t)(warps + 1) * experts * sizeof(float);
    const dim3 grid(n);
    if (dtype == DE_BF16)
        return de_launch(route_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, s,
                         (const __nv_bfloat16*)h, ldh, w, bias, n, width, experts, top, mode,
                         chosen, weight);
    return de_launch(route_kernel<float>, grid, dim3(warps * 32), smem, s, (const float*)h, ldh, w,
                     bias, n, width, experts, top, mode, chosen, weight);
}

DE_EXPORT int de_experts_group(const int* chosen, int pairs, int experts, int tiles, int seg,
                               int* pair_of, int* tile_expert, int* slot_of, void* stream) {
    if (pairs <= 0) return 0;
    if (experts > 4096 || seg <= 0) return -2;
    return de_launch(group_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int),
                     (cudaStream_t)stream, chosen, pairs, experts, tiles, seg, pair_of,
                     tile_expert, slot_of);
}

// rows[slot] = h[token of the slot's pair] (zeros for a slot without a pair): the operand of the
// tensor-core product, whose tiles are rows of one expert.
DE_EXPORT int de_experts_gather(int dtype, const void* h, int ldh, const int* pair_of, int slots,
                                int top, int width, void* rows, void* stream) {
    if (slots <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16)
        return de_launch(gather_kernel<__nv_bfloat16>, dim3(slots), dim3(128), 0, s,
                         (const __nv_bfloat16*)h, ldh, pair_of, top, width, (__nv_bfloat16*)rows);
    return de_launch(gather_kernel<float>, dim3(slots), dim3(128), 0, s, (const float*)h, ldh,
                     pair_of, top, width, (float*)rows);
}

DE_EXPORT int de_experts_up(int dtype, const void* h, int ldh, const void* up, const int* pair_of,
                            const int* tile_expert, int tiles, int top, int width, int ff,
                            void* inner, int act, void* stream) {
    if (tiles <= 0) return 0;
    if (act < 0 || act > 5) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int size = dtype == DE_BF16 ? 2 : 4;
    const int vec_a = ((uintptr_t)h % (4 * size) == 0) && ldh % 4 == 0;
    const int vec_w = ((uintptr_t)up % (4 * size) == 0) && width % 4 == 0;
    const dim3 grid(tiles, (ff + rows_product::TILE - 1) / rows_product::TILE);
    if (grid.y > 65535) return -2;
    if (dtype == DE_BF16)
        return de_launch(expert_up_kernel<__nv_bfloat16>, grid, dim3(rows_product::THREADS), 0, s,
                         (const __nv_bfloat16*)h, ldh, (const __nv_bfloat16*)up, pair_of,
                         tile_expert, top, width, ff, (__nv_bfloat16*)inner, act, vec_a, vec_w);
    return de_launch(expert_up_kernel<float>, grid, dim3(rows_product::THREADS), 0, s,
                     (const float*)h, ldh, (const float*)up, pair_of, tile_expert, top, width, ff,
                     (float*)inner, act, vec_a, vec_w);
}

DE_EXPORT int de_experts_down(int dtype, const void* inner, const void* down, const int* pair_of,
                              const int* tile_expert, int tiles, int width, int ff, void* y,
                              void* stream) {
    if (tiles <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int size = dtype == DE_BF16 ? 2 : 4;
    const int vec_a = ((uintptr_t)inner % (4 * size) == 0) && ff % 4 == 0;
    const int vec_w = ((uintptr_t)down % (4 * size) == 0) && ff % 4 == 0;
    const dim3 grid(tiles, (width + rows_product::TILE - 1) / rows_product::TILE);
    if (grid.y > 65535) return -2;
    if (dtype == DE_BF16)
        return de_launch(expert_down_kernel<__nv_bfloat16>, grid, dim3(rows_product::THREADS), 0,
                         s, (const __nv_bfloat16*)inner, (const __nv_bfloat16*)down, pair_of,
                         tile_expert, width, ff, (__nv_bfloat16*)y, vec_a, vec_w);
    return de_launch(expert_down_kernel<float>, grid, dim3(rows_product::THREADS), 0, s,
                     (const float*)inner, (const float*)down, pair_of, tile_expert, width, ff,
                     (float*)y, vec_a, vec_w);
}

DE_EXPORT int de_experts_combine(int dtype, const void* y, const float* weight, int n, int top,
                                 int width, float* out, const int* chosen, int experts,
                                 const void* h, int ldh, void* stream) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16)
        return de_launch(combine_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, s,
                         (const __nv_bfloat16*)y, weight, top, width, total, out, chosen, experts,
                         (const __nv_bfloat16*)h, ldh);
    return de_launch(combine_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s,
                     (const float*)y, weight, top, width, total, out, chosen, experts,
                     (const float*)h, ldh);
}
