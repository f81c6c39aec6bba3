// Softmax attention inside chunks of positions, over the paged cache, with a penalty that grows
// with the logarithm of the distance, keys and values of different sizes, and values that are
// cached normalised.  Float32 arithmetic on the CUDA cores for float32 or bfloat16 storage:
// scores, the penalty, the softmax weights and the weighted sum of the values are all 32-bit.
//
//   score(i, j) = (q_i . k_j) * scale - r1[h] * log(1 + r2[h] * (i - j))
//   token i sees key j when j <= i and floor(i / chunk) = floor(j / chunk)   (chunks of positions
//   counted from 0 of the sequence, whatever portion of it a step brings)
//
// A row is (token, query head within its kv head's group); a block takes a tile of 8 rows of one
// sequence and one kv head, a warp a row, a lane a key of the current tile of 32 keys.  Tiles of
// keys lie at absolute multiples of 32 and a row walks the tiles of its chunk in ascending order,
// so a row's result does not depend, bit for bit, on what shares its tile, its step or its batch.
// The host's work items are those of the other attention kernels (kernels/attention_plan.py),
// unsplit: a chunk bounds every key range.
//
// The same kernels also serve attention whose keys are bounded by a sliding window that keeps the
// first tokens of the sequence, with a soft cap on the scores (`Sight`):
//
//   token i sees key j when j <= i and (i - j < window or j < keep_first)
//   score <- softcap * tanh(score / softcap)
//
// A block then walks the tiles of the kept first keys and jumps to the tile in which its rows'
// windows begin.  r1 / r2 null: no distance penalty.  `out_f32`: the rows' results are written as
// float32 (for a kernel that turns them by position or gates them before they are rounded).
//
// Three more parameters of `Sight` serve attention whose softmax has a sink: a distance penalty
// that is linear, r1[h] * (i - j); `sink` [heads], a learned score per head that joins the
// denominator as exp(sink[h]) without a key or a value (it is added once, when a row's sums are
// complete, whatever the tiles and the step's cut); and `gate`, sigmoid of which multiplies a
// row's result in float32 before it is stored (one number a feature or one a head).  qkv_prepare
// is what stands between such a mixer's projection and these kernels (bias, a short convolution
// over time with the slot's kept rows, norms, rotation, value mixing, the cache write), and
// conv_keep moves the kept rows on.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int ROWS = 8;
constexpr int TILE = 32;
constexpr int MAX_D = 256;        // of a value: the weighted sums live in registers
constexpr int MAX_DK = 576;       // of a key: shared memory only

struct WorkItem {
    int seq, row0, kv_begin, kv_end, partial, pad0, pad1, pad2;
};

// Which keys a row sees besides j <= i, and what happens to its scores.
struct Sight {
    int chunk;          // > 0: keys of the row's own chunk of positions only
    int window;         // > 0: the last `window` keys only ...
    int keep_first;     // ... and the first `keep_first` keys of the sequence
    float softcap;      // > 0: score <- softcap * tanh(score / softcap)
    int v_stride;       // elements from one key's values to the next in v_pages: dv, or the key
                        // size where the values are the first dv features of the key rows
    int linear;         // the distance penalty is r1[h] * (i - j) instead of the logarithmic one
    const float* sink;  // [heads] or null: the softmax's denominator also holds exp(sink[h]), a
                        // weight without a key or a value (not scaled, no penalty)
    const void* gate;   // or null: a row's result is multiplied by sigmoid(gate) before it is
    int ld_gate;        // stored; gate of the queries' type, rows ld_gate apart, one number a
    int gate_per_head;  // feature ([heads dv]) or, with gate_per_head, one a head ([heads])
};
template <typename T>
__device__ __forceinline__ float sight_gate(const Sight& s, size_t token, int head, int dv,
                                            int feature) {
    if (s.gate == nullptr) return 1.0f;
    const T* g = (const T*)s.gate + token * s.ld_gate + (s.gate_per_head ? head : head * dv + feature);
    return 1.0f / (1.0f + expf(-to_float(*g)));
}
// 1 / (the row's sum of weights, with the sink's share): m is the row's reference maximum
__device__ __forceinline__ float sight_inverse(const Sight& s, int head, float m, float l) {
    if (s.sink != nullptr) l += expf(s.sink[head] - m);
    return l > 0.0f ? 1.0f / l : 0.0f;
}

// first key of the near range of a row at `pos` (does not fall as pos grows)
__device__ __forceinline__ int sight_lo(const Sight& m, int pos) {
    int lo = 0;
    if (m.chunk > 0) lo = pos / m.chunk * m.chunk;
    if (m.window > 0) lo = max(lo, pos - m.window + 1);
    return lo;
}
// keys [0, this) are seen as well
__device__ __forceinline__ int sight_first(const Sight& m, int lo) {
    return (m.window > 0 && m.keep_first > 0) ? min(m.keep_first, lo) : 0;
}
__device__ __forceinline__ float sight_score(const Sight& m, float s, float scale, float pen1,
                                             float pen2, bool penalty, float dist) {
    s *= scale;
    if (penalty) s -= m.linear ? pen1 * dist : pen1 * log1pf(pen2 * dist);
    if (m.softcap > 0.0f) s = m.softcap * tanhf(s / m.softcap);
    return s;
}
// The tiles a block walks: those of the kept first keys [0, kf), then from the tile of `lo` on.
struct TileWalk {
    int start, jump_at, jump_to;
    __device__ __forceinline__ TileWalk(int lo, int kf, int tile) {
        const int near = (lo / tile) * tile, first_end = ((kf + tile - 1) / tile) * tile;
        start = kf > 0 ? 0 : near;
        jump_at = (kf > 0 && first_end < near) ? first_end : -1;
        jump_to = near;
    }
    __device__ __forceinline__ int next(int kt, int tile) const {
        const int n = kt + tile;
        return n == jump_at ? jump_to : n;
    }
};
template <typename T>
__device__ __forceinline__ void store_out(void* out, int out_f32, size_t at, float x) {
    if (out_f32) ((float*)out)[at] = x;
    else ((T*)out)[at] = from_float<T>(x);
}

// k copied, v divided by its root mean square over the head (eps inside the root), both into the
// pages.  proj row = [... | k (G dk) | v (G dv)] from column k_col on.  grid (tokens, kv heads).
template <typename T>
__global__ void kv_write_normed_kernel(const T* __restrict__ proj, int ld, int k_col,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ token_slot, int G, int dk, int dv,
                                       float eps, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                       const int* __restrict__ block_table, int table_stride,
                                       int page, int num_pages, int* __restrict__ status) {
    __shared__ float scratch[33];
    const int n = blockIdx.x, hk = blockIdx.y;
    const int pos = positions[n], slot = token_slot[n];
    pdl_wait();
    const int page_id = block_table[(size_t)slot * table_stride + pos / page];
    const T* ks = proj + (size_t)n * ld + k_col + hk * dk;
    const T* vs = proj + (size_t)n * ld + k_col + G * dk + hk * dv;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        const float x = to_float(vs[i]);
        ss = fmaf(x, x, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dv + eps);
    pdl_trigger();
    if (page_id < 0 || page_id >= num_pages) {       // never written outside the pool
        if (threadIdx.x == 0) atomicExch(status, 1);
        return;
    }
    const size_t at = ((size_t)page_id * G + hk) * page + (size_t)(pos % page);
    for (int i = threadIdx.x; i < dk; i += blockDim.x) k_pages[at * dk + i] = ks[i];
    for (int i = threadIdx.x; i < dv; i += blockDim.x)
        v_pages[at * dv + i] = from_float<T>(to_float(vs[i]) * inv);
}

// Queries and keys turned by position, values turned by position over all their features, keys
// and values into the pages.  proj row = [q (H dk) | k (G dk) | v (G dv) | ...] (a run that reads
// another run's cache has q only: write_kv 0).  Pairs are (i, i + n/2) of the first n features:
// n = rot with the angles pos * fk[i] for q and k, n = dv with pos * fv[i] for v (fv null: values
// are stored as they are).  q is turned in place.  One block a token.
template <typename T>
__global__ void kv_write_rotated_kernel(T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                        const int* __restrict__ token_slot,
                                        const float* __restrict__ fk, int rot,
                                        const float* __restrict__ fv, int H, int G, int dk, int dv,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages,
                                        const int* __restrict__ block_table, int table_stride,
                                        int page, int num_pages, int write_kv,
                                        int* __restrict__ status) {
    const int n = blockIdx.x;
    const int pos = positions[n];
    const float fpos = (float)pos;
    T* row = proj + (size_t)n * ld;
    const int half = rot / 2, per = dk - half;       // work items a head: pairs, then plain features
    size_t at = 0;
    bool can_write = write_kv != 0;
    if (can_write) {
        const int page_id = block_table[(size_t)token_slot[n] * table_stride + pos / page];
        if (page_id < 0 || page_id >= num_pages) {   // never written outside the pool
            if (threadIdx.x == 0) atomicExch(status, 1);
            can_write = false;
        }
        at = ((size_t)page_id * G) * page + (size_t)(pos % page);
    }
    pdl_wait();
    const int qk_heads = H + (write_kv ? G : 0);
    for (int idx = threadIdx.x; idx < qk_heads * per; idx += blockDim.x) {
        const int h = idx / per, i = idx - h * per;
        T* src = row + h * dk;
        T* dst = src;                                // q in place
        if (h >= H) {
            if (!can_write) continue;
            dst = k_pages + (at + (size_t)(h - H) * page) * dk;
        }
        if (i < half) {
            float sn, cs, ra, rb;
            sincosf(fpos * fk[i], &sn, &cs);
            rope_rotate(to_float(src[i]), to_float(src[i + half]), cs, sn, ra, rb);
            dst[i] = from_float<T>(ra);
            dst[i + half] = from_float<T>(rb);
        } else if (h >= H) {
            dst[i + half] = src[i + half];
        }
    }
    if (can_write) {
        const T* vs = row + (H + G) * dk;
        if (fv != nullptr) {
            const int vhalf = dv / 2, vper = dv - vhalf;
            for (int idx = threadIdx.x; idx < G * vper; idx += blockDim.x) {
                const int h = idx / vper, i = idx - h * vper;
                const T* src = vs + h * dv;
                T* dst = v_pages + (at + (size_t)h * page) * dv;
                if (i < vhalf) {
                    float sn, cs, ra, rb;
                    sincosf(fpos * fv[i], &sn, &cs);
                    rope_rotate(to_float(src[i]), to_float(src[i + vhalf]), cs, sn, ra, rb);
                    dst[i] = from_float<T>(ra);
                    dst[i + vhalf] = from_float<T>(rb);
                } else {
                    dst[i + vhalf] = src[i + vhalf];
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
                const int h = idx / dv, i = idx - h * dv;
                v_pages[(at + (size_t)h * page) * dv + i] = vs[idx];
            }
        }
    }
    pdl_trigger();
}

// What lies between a mixer's stacked projection and its attention, for mixers that do more to
// q, k and v than turn them: proj row = [q (H dk) | k (G dk) | v (G dv) | ...], C = (H + G) dk +
// G dv channels.  In this order, each step optional:
//   bias      u = proj + bias[c]
//   taps      a short causal convolution over time on every channel, y_t = sum_j taps[c][j] *
//             u_(t - K + 1 + j), zeros before the sequence's start; inputs before the step's first
//             token of the sequence come from the slot's state, kept[i] = projection (without
//             bias) at position pos0 - (K - 1) + i, as conv_keep leaves them; with keep_here (a
//             step in which every sequence brings one token, so no other block reads the
//             slot) the block moves the kept rows on itself and conv_keep is not needed
//   norm      q and k divided by their root mean square (eps inside the root) and weighted: 1 over
//             every head with weights [dk] that all heads share, 2 over the whole projection with
//             weights [H dk] and [G dk]
//   freq      the first `rot` features of every head of q and k turned by position, angle = pos *
//             freq[i] (formed in double precision), cosine and sine times `magnitude`; pairs are
//             (2i, 2i + 1) with `adjacent`, else (i, i + rot / 2)
//   temp      q times 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
//   mix       1: the values (as they are cached) are also left in v_first [N, G dv];
//             2: v <- (1 - lambda) v + lambda v_first, lambda one number on the device
// q goes to q_out [N, H dk] in the activation type, k and v into the pages.  All arithmetic is
// float32.  One block a token; shared memory: C + rot + H + G floats.
struct Prepare {
    const float* bias;
    const float* taps;
    int K;
    float* state;
    long long slot_stride;
    int conv_offset;
    int norm;
    const float* q_weight;
    const float* k_weight;
    float eps;
    const float* freq;
    int rot;
    float magnitude;
    int adjacent;
    float temp_coef;
    int temp_every;
    int mix;
    const float* lambda;
    float* v_first;
    int keep_here;
};

// 16 bytes of the projection as floats
__device__ __forceinline__ void load_piece(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load_piece(const __nv_bfloat16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// two neighbouring features in one store
__device__ __forceinline__ void store_pair(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
// Two sums over a block at once; every thread gets both.  The order of the additions depends on
// the block's size only.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch /* 66 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
        scratch[warp] = a;
        scratch[32 + warp] = b;
    }
    __syncthreads();
    if (warp < 2) {
        float t = lane < warps ? scratch[32 * warp + lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[64 + warp] = t;
    }
    __syncthreads();
    a = scratch[64];
    b = scratch[65];
}

// VEC: the rows of proj are whole 16-byte pieces at 16-byte addresses and C is a whole number of
// pieces; a thread then takes the convolution of a piece's channels at once.  The sums are the
// same chains of multiply-adds either way.
template <typename T, bool VEC>
__global__ void qkv_prepare_kernel(const T* __restrict__ proj, int ld, T* __restrict__ q_out,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ token_seq,
                                   const int* __restrict__ token_slot,
                                   const int* __restrict__ seq_pos0, Prepare pp, int H, int G,
                                   int dk, int dv, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                   const int* __restrict__ block_table, int table_stride, int page,
                                   int num_pages, int* __restrict__ status) {
    extern __shared__ float sh[];
    __shared__ float scratch[66];
    const int n = blockIdx.x;
    const int qk = (H + G) * dk, C = qk + G * dv, half = pp.rot / 2;
    float* cs_tab = sh + C;                          // [half] cosines, then [half] sines
    float* inv_s = cs_tab + pp.rot;                  // [H + G]
    const int pos = positions[n], slot = token_slot[n];
    const int off = pos - seq_pos0[token_seq[n]];    // the token's place in its sequence's portion
    const int page_id = block_table[(size_t)slot * table_stride + pos / page];
    const bool can_write = page_id >= 0 && page_id < num_pages;
    if (!can_write && threadIdx.x == 0) atomicExch(status, 1);   // never written outside the pool
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double sn, cs;
        sincos((double)pos * (double)pp.freq[i], &sn, &cs);
        cs_tab[i] = (float)cs * pp.magnitude;
        cs_tab[half + i] = (float)sn * pp.magnitude;
    }
    pdl_wait();
    const T* row = proj + (size_t)n * ld;
    if (VEC && pp.taps != nullptr && pp.K > 1) {
        constexpr int PN = 16 / (int)sizeof(T);
        const int K = pp.K;
        const float* kept = pp.state + (size_t)slot * pp.slot_stride + pp.conv_offset;
        for (int c0 = threadIdx.x * PN; c0 < C; c0 += blockDim.x * PN) {
            float acc[PN], b[PN];
#pragma unroll
            for (int e = 0; e < PN; ++e) {
                acc[e] = 0.0f;
                b[e] = pp.bias ? pp.bias[c0 + e] : 0.0f;
            }
            for (int j = 0; j < K; ++j) {
                const int rel = off - (K - 1) + j;
                if (pos - (K - 1) + j < 0) continue;             // before the sequence's start
                float x[PN];
                if (rel >= 0) {
                    load_piece(proj + (size_t)(n - (K - 1) + j) * ld + c0, x);
                } else {
#pragma unroll
                    for (int e = 0; e < PN; ++e) x[e] = kept[(size_t)(off + j) * C + c0 + e];
                }
#pragma unroll
                for (int e = 0; e < PN; ++e)
                    acc[e] = fmaf(pp.taps[(c0 + e) * K + j], x[e] + b[e], acc[e]);
            }
#pragma unroll
            for (int e = 0; e < PN; ++e) sh[c0 + e] = acc[e];
        }
    } else if (pp.taps != nullptr && pp.K > 1) {
        const int K = pp.K;
        const float* kept = pp.state + (size_t)slot * pp.slot_stride + pp.conv_offset;
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            const float b = pp.bias ? pp.bias[c] : 0.0f;
            float acc = 0.0f;
            for (int j = 0; j < K; ++j) {
                const int rel = off - (K - 1) + j;
                if (pos - (K - 1) + j < 0) continue;             // before the sequence's start
                const float x = rel >= 0 ? to_float(proj[(size_t)(n - (K - 1) + j) * ld + c])
                                         : kept[(size_t)(off + j) * C + c];
                acc = fmaf(pp.taps[c * K + j], x + b, acc);
            }
            sh[c] = acc;
        }
    } else if (VEC) {
        constexpr int PN = 16 / (int)sizeof(T);
        for (int c0 = threadIdx.x * PN; c0 < C; c0 += blockDim.x * PN) {
            float x[PN];
            load_piece(row + c0, x);
#pragma unroll
            for (int e = 0; e < PN; ++e) {
                x[e] += pp.bias ? pp.bias[c0 + e] : 0.0f;
                sh[c0 + e] = pp.taps != nullptr ? pp.taps[c0 + e] * x[e] : x[e];   // one tap
            }
        }
    } else {
        const float tap = pp.taps != nullptr ? 1.0f : 0.0f;     // a convolution of one tap
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            const float x = to_float(row[c]) + (pp.bias ? pp.bias[c] : 0.0f);
            sh[c] = tap != 0.0f ? pp.taps[c] * x : x;
        }
    }
    __syncthreads();
    if (pp.keep_here && pp.taps != nullptr && pp.K > 1) {
        // every thread has read what it needs of the kept rows; a thread moves its channels on
        float* kept = pp.state + (size_t)slot * pp.slot_stride + pp.conv_offset;
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            for (int i = 0; i + 2 < pp.K; ++i) kept[(size_t)i * C + c] = kept[(size_t)(i + 1) * C + c];
            kept[(size_t)(pp.K - 2) * C + c] = to_float(row[c]);
        }
    }
    if (pp.norm == 1) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int h = warp; h < H + G; h += warps) {
            float ss = 0.0f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(sh[h * dk + i], sh[h * dk + i], ss);
            ss = warp_sum(ss);
            if (lane == 0) inv_s[h] = 1.0f / sqrtf(ss / (float)dk + pp.eps);
        }
    } else if (pp.norm == 2) {
        float sq = 0.0f, sk = 0.0f;
        for (int i = threadIdx.x; i < H * dk; i += blockDim.x) sq = fmaf(sh[i], sh[i], sq);
        for (int i = H * dk + threadIdx.x; i < qk; i += blockDim.x) sk = fmaf(sh[i], sh[i], sk);
        block_sum2(sq, sk, scratch);
        const float iq = 1.0f / sqrtf(sq / (float)(H * dk) + pp.eps);
        const float ik = 1.0f / sqrtf(sk / (float)(G * dk) + pp.eps);
        for (int h = threadIdx.x; h < H + G; h += blockDim.x) inv_s[h] = h < H ? iq : ik;
    }
    __syncthreads();
    pdl_trigger();
    float temp = 1.0f;
    if (pp.temp_every > 0) temp = 1.0f + pp.temp_coef * logf((float)((pos + 1) / pp.temp_every) + 1.0f);
    const size_t at = ((size_t)(can_write ? page_id : 0) * G) * page + (size_t)(pos % page);
    const bool paired = dk % 2 == 0 && (pp.adjacent || half == 0);
    // neighbouring features two at a time (turned together, or both plain), one store for both
    for (int idx = threadIdx.x; idx < (paired ? (H + G) * (dk / 2) : 0); idx += blockDim.x) {
        const int h = idx / (dk / 2), i = idx - h * (dk / 2);
        const bool is_q = h < H;
        if (!is_q && !can_write) continue;
        const float* x = sh + h * dk;
        const float* wt = nullptr;
        float inv = 1.0f;
        if (pp.norm != 0) {
            inv = inv_s[h];
            wt = is_q ? pp.q_weight : pp.k_weight;
            if (pp.norm == 2) wt += (is_q ? h : h - H) * dk;
        }
        const float mul = is_q ? temp : 1.0f;
        T* dst = is_q ? q_out + (size_t)n * (H * dk) + h * dk
                      : k_pages + (at + (size_t)(h - H) * page) * dk;
        const int a = 2 * i, b = a + 1;
        float ra = x[a] * inv * (wt ? wt[a] : 1.0f), rb = x[b] * inv * (wt ? wt[b] : 1.0f);
        if (i < half) rope_rotate(ra, rb, cs_tab[i], cs_tab[half + i], ra, rb);
        store_pair(dst + a, ra * mul, rb * mul);
    }
    const int per = dk - half;                       // work items a head: pairs, then plain features
    for (int idx = threadIdx.x; idx < (paired ? 0 : (H + G) * per); idx += blockDim.x) {
        const int h = idx / per, i = idx - h * per;
        const bool is_q = h < H;
        if (!is_q && !can_write) continue;
        const float* x = sh + h * dk;
        const float* wt = nullptr;
        float inv = 1.0f;
        if (pp.norm != 0) {
            inv = inv_s[h];
            wt = is_q ? pp.q_weight : pp.k_weight;
            if (pp.norm == 2) wt += (is_q ? h : h - H) * dk;
        }
        const float mul = is_q ? temp : 1.0f;
        T* dst = is_q ? q_out + (size_t)n * (H * dk) + h * dk
                      : k_pages + (at + (size_t)(h - H) * page) * dk;
        if (i < half) {
            const int a = pp.adjacent ? 2 * i : i, b = pp.adjacent ? 2 * i + 1 : i + half;
            float ra, rb;
            rope_rotate(x[a] * inv * (wt ? wt[a] : 1.0f), x[b] * inv * (wt ? wt[b] : 1.0f),
                        cs_tab[i], cs_tab[half + i], ra, rb);
            dst[a] = from_float<T>(ra * mul);
            dst[b] = from_float<T>(rb * mul);
        } else {
            const int a = i + half;
            dst[a] = from_float<T>(x[a] * inv * (wt ? wt[a] : 1.0f) * mul);
        }
    }
    const float lam = pp.mix == 2 ? pp.lambda[0] : 0.0f;
    for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
        float v = sh[qk + idx];
        if (pp.mix == 2) v = (1.0f - lam) * v + lam * pp.v_first[(size_t)n * (G * dv) + idx];
        const T stored = from_float<T>(v);
        if (pp.mix == 1) pp.v_first[(size_t)n * (G * dv) + idx] = to_float(stored);
        if (can_write) {
            const int h = idx / dv, i = idx - h * dv;
            v_pages[(at + (size_t)h * page) * dv + i] = stored;
        }
    }
}

// After qkv_prepare: every sequence's slot keeps the last K - 1 rows of the first C columns of
// proj (the convolution's inputs of the next step), kept[i] = the row at position
// pos0 + qlen - (K - 1) + i; a portion shorter than K - 1 moves the older rows up.  The layout is
// the one that the state mixers' convolution keeps (recurrent.cu); a model whose only
// convolution is this mixer's needs no other library for it.  One block a sequence.
template <typename T>
__global__ void conv_keep_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state,
                                 long long slot_stride, int conv_offset,
                                 const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_qstart,
                                 const int* __restrict__ seq_qlen, int C, int K) {
    const int s = blockIdx.x;
    const int qlen = seq_qlen[s], tok0 = seq_qstart[s];
    pdl_wait();
    pdl_trigger();
    float* kept = state + (size_t)seq_slot[s] * slot_stride + conv_offset;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        for (int i = 0; i < K - 1; ++i) {            // ascending: what is read lies ahead
            const int rel = qlen - (K - 1) + i;
            kept[(size_t)i * C + c] = rel >= 0 ? to_float(proj[(size_t)(tok0 + rel) * ld + c])
                                               : kept[(size_t)(i + qlen) * C + c];
        }
}

// After the attention: every head's result (float32 [N, H dv]) turned back by its token's position
// (pairs (i, i + dv/2), angle -pos * fv[i]; fv null: as it is), times sigmoid(gate) where a gate
// (type T, row stride ld_gate; one number a feature, or one a head with gate_per_head) is given,
// rounded to the activation type.  One block a token.
template <typename T>
__global__ void attn_finish_kernel(const float* __restrict__ o, const int* __restrict__ positions,
                                   const float* __restrict__ fv, const T* __restrict__ gate,
                                   int ld_gate, T* __restrict__ out, int H, int dv,
                                   int gate_per_head) {
    const int n = blockIdx.x;
    const float fpos = (float)positions[n];
    const float* src = o + (size_t)n * H * dv;
    T* dst = out + (size_t)n * H * dv;
    const T* gt = gate ? gate + (size_t)n * ld_gate : nullptr;
    pdl_wait();
    pdl_trigger();
    if (fv != nullptr) {
        const int half = dv / 2, per = dv - half;
        for (int idx = threadIdx.x; idx < H * per; idx += blockDim.x) {
            const int h = idx / per, i = idx - h * per;
            const int a = h * dv + i, b = a + half;
            if (i < half) {
                float sn, cs, ra, rb;
                sincosf(fpos * fv[i], &sn, &cs);
                rope_rotate(src[a], src[b], cs, -sn, ra, rb);
                if (gt) {
                    ra *= 1.0f / (1.0f + expf(-to_float(gt[gate_per_head ? h : a])));
                    rb *= 1.0f / (1.0f + expf(-to_float(gt[gate_per_head ? h : b])));
                }
                dst[a] = from_float<T>(ra);
                dst[b] = from_float<T>(rb);
            } else {
                float x = src[b];
                if (gt) x *= 1.0f / (1.0f + expf(-to_float(gt[gate_per_head ? h : b])));
                dst[b] = from_float<T>(x);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < H * dv; idx += blockDim.x) {
            float x = src[idx];
            if (gt) x *= 1.0f / (1.0f + expf(-to_float(gt[gate_per_head ? idx / dv : idx])));
            dst[idx] = from_float<T>(x);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(ROWS * 32)
attn_chunk_kernel(const T* __restrict__ q, int q_stride, void* __restrict__ out, int out_stride,
                  const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                  const int* __restrict__ block_table, int table_stride, int num_pages,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                  const int* __restrict__ seq_qlen, const int* __restrict__ seq_pos0,
                  const WorkItem* __restrict__ items, const float* __restrict__ r1,
                  const float* __restrict__ r2, int heads, int kv_heads, int dk, int dv, int page,
                  float scale, Sight sight, int out_f32, int* __restrict__ status) {
    extern __shared__ float smem[];
    float* Ks = smem;                       // [TILE][dk + 1]; column dk: 0, or -inf without a page
    float* Vs = Ks + TILE * (dk + 1);       // [TILE][dv]
    float* Qs = Vs + TILE * dv;             // [ROWS][dk]

    const WorkItem it = items[blockIdx.x];
    if (it.kv_begin >= it.kv_end) {
        pdl_wait();
        return;
    }
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int r = it.row0 + warp;
    const bool active = r < rows_total;
    const int t = active ? r / g : 0;
    const int hq = hk * g + (active ? r % g : 0);
    const int pos = pos0 + t;
    const bool penalty = r1 != nullptr;
    const float pen1 = penalty ? r1[hq] : 0.0f, pen2 = penalty ? r2[hq] : 0.0f;

    pdl_wait();
    for (int i = lane; i < dk; i += 32)
        Qs[warp * dk + i] = active ? to_float(q[(size_t)(tok0 + t) * q_stride + hq * dk + i]) : 0.0f;

    // the tile's key range: from the chunk or window of its first token to its last token, and
    // the kept first keys
    const int last_row = min(it.row0 + ROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    const int k_lo_true = max(it.kv_begin, sight_lo(sight, min_pos));
    const int k_first = it.kv_begin > 0 ? 0 : sight_first(sight, k_lo_true);
    const TileWalk walk(k_lo_true, k_first, TILE);
    // this row's
    const int row_lo = max(it.kv_begin, sight_lo(sight, pos));
    const int row_first = it.kv_begin > 0 ? 0 : sight_first(sight, row_lo);
    const int row_hi = min(it.kv_end, pos + 1);

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.0f;

    for (int kt = walk.start; kt < k_hi; kt = walk.next(kt, TILE)) {
        __syncthreads();
        for (int j = warp; j < TILE; j += ROWS) {        // a warp a key: whole rows of the pages
            const int kpos = kt + j;
            bool held = true, inside = (kpos >= k_lo_true || kpos < k_first) && kpos < k_hi;
            size_t at = 0;
            if (inside) {
                const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
                held = page_id >= 0 && page_id < num_pages;
                at = ((size_t)page_id * kv_heads + hk) * page + (size_t)(kpos % page);
            }
            const bool read = inside && held;
            for (int i = lane; i < dk; i += 32)
                Ks[j * (dk + 1) + i] = read ? to_float(k_pages[at * dk + i]) : 0.0f;
            for (int i = lane; i < dv; i += 32)
                Vs[j * dv + i] = read ? to_float(v_pages[at * sight.v_stride + i]) : 0.0f;
            if (lane == 0) {
                Ks[j * (dk + 1) + dk] = held ? 0.0f : -INFINITY;
                if (!held && status != nullptr) atomicExch(status, 2);
            }
        }
        __syncthreads();
        if (!active) continue;

        const int kpos = kt + lane;
        const float* kr = Ks + lane * (dk + 1);
        const bool valid = (kpos >= row_lo || kpos < row_first) && kpos < row_hi && kr[dk] == 0.0f;
        const float* qr = Qs + warp * dk;
        float s = 0.0f;
        for (int i = 0; i < dk; ++i) s = fmaf(qr[i], kr[i], s);
        s = valid ? sight_score(sight, s, scale, pen1, pen2, penalty, (float)(pos - kpos)) : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
        for (int j = 0; j < TILE; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.0f) continue;
            const float* vr = Vs + j * dv;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int dd = lane + 32 * i;
                if (dd < dv) acc[i] = fmaf(pj, vr[dd], acc[i]);
            }
        }
        m = m_new;
    }
    pdl_trigger();
    if (!active) return;
    const float inv = sight_inverse(sight, hq, m, l);
    const size_t o = (size_t)(tok0 + t) * out_stride + hq * dv;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int dd = lane + 32 * i;
        if (dd < dv)
            store_out<T>(out, out_f32, o + dd,
                         acc[i] * inv * sight_gate<T>(sight, (size_t)(tok0 + t), hq, dv, dd));
    }
}


// ------------------------------------------------------------------------------------------
// The same attention for key and value rows that are whole 16-byte pieces (sizes that are a
// multiple of 8 in bfloat16, of 4 in float32): the next tile of keys and values is asked for in
// 16-byte loads into registers before the current one is worked on, a warp takes RW rows (it
// reads a key or a value from shared memory once for all of them), and shared memory is read as
// float4.  A row's sums are formed in the same order as in the kernel above whatever RW is.
// ------------------------------------------------------------------------------------------
template <typename T> struct Piece;                 // 16 bytes of T as floats
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
};
template <> struct Piece<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T, int RW, int NCH>
__global__ void __launch_bounds__(ROWS * 32, NCH <= 4 ? 2 : 1)
attn_chunk_vec_kernel(const T* __restrict__ q, int q_stride, void* __restrict__ out, int out_stride,
                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      const int* __restrict__ block_table, int table_stride, int num_pages,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                      const int* __restrict__ seq_qlen, const int* __restrict__ seq_pos0,
                      const WorkItem* __restrict__ items, const float* __restrict__ r1,
                      const float* __restrict__ r2, int heads, int kv_heads, int dk, int dv,
                      int page, float scale, Sight sight, int out_f32, int* __restrict__ status) {
    constexpr int PN = Piece<T>::N;
    extern __shared__ __align__(16) float smem[];
    const int ks = ((dk + 31) / 32) * 32 + 4;       // a key's stride: float4 reads without conflicts
    float* Ks = smem;                                // [TILE][ks]
    float* Vs = Ks + TILE * ks;                      // [TILE][dv]
    float* Qs = Vs + TILE * dv;                      // [ROWS * RW][dk]
    float* Held = Qs + ROWS * RW * dk;               // [TILE]: 0, or -inf for a key without a page

    const WorkItem it = items[blockIdx.x];
    if (it.kv_begin >= it.kv_end) {
        pdl_wait();
        return;
    }
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    bool active[RW];
    int tok[RW], hq[RW], pos[RW], row_lo[RW], row_hi[RW], row_first[RW];
    float pen1[RW], pen2[RW], m[RW], l[RW];
    bool any = false;
    const bool penalty = r1 != nullptr;
#pragma unroll
    for (int i = 0; i < RW; ++i) {
        const int r = it.row0 + warp * RW + i;
        active[i] = r < rows_total;
        any |= active[i];
        tok[i] = active[i] ? r / g : 0;
        hq[i] = hk * g + (active[i] ? r % g : 0);
        pos[i] = pos0 + tok[i];
        pen1[i] = penalty ? r1[hq[i]] : 0.0f;
        pen2[i] = penalty ? r2[hq[i]] : 0.0f;
        row_lo[i] = max(it.kv_begin, sight_lo(sight, pos[i]));
        row_first[i] = it.kv_begin > 0 ? 0 : sight_first(sight, row_lo[i]);
        row_hi[i] = min(it.kv_end, pos[i] + 1);
        m[i] = -INFINITY;
        l[i] = 0.0f;
    }
    const int last_row = min(it.row0 + ROWS * RW, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    const int k_lo_true = max(it.kv_begin, sight_lo(sight, min_pos));
    const int k_first = it.kv_begin > 0 ? 0 : sight_first(sight, k_lo_true);
    const TileWalk walk(k_lo_true, k_first, TILE);

    const int ck = dk / PN, cv = dv / PN, per_key = ck + cv;
    uint4 pre[NCH];
    unsigned missing = 0;                            // bit c: piece c's key has no page

    pdl_wait();
    auto prefetch = [&](int kt) {
        missing = 0;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int e = threadIdx.x + c * (ROWS * 32);
            pre[c] = make_uint4(0u, 0u, 0u, 0u);
            if (e >= TILE * per_key) continue;
            const int j = e / per_key, w = e - j * per_key;
            const int kpos = kt + j;
            if ((kpos < k_lo_true && kpos >= k_first) || kpos >= k_hi) continue;
            const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
            if (page_id < 0 || page_id >= num_pages) {
                missing |= 1u << c;
                continue;
            }
            const size_t at = ((size_t)page_id * kv_heads + hk) * page + (size_t)(kpos % page);
            const T* src = w < ck ? k_pages + at * dk + w * PN : v_pages + at * sight.v_stride + (w - ck) * PN;
            pre[c] = *reinterpret_cast<const uint4*>(src);
        }
    };
    prefetch(walk.start);
#pragma unroll
    for (int i = 0; i < RW; ++i)
        for (int d = lane; d < dk; d += 32)
            Qs[(warp * RW + i) * dk + d] =
                active[i] ? to_float(q[(size_t)(tok0 + tok[i]) * q_stride + hq[i] * dk + d]) : 0.0f;

    float acc[RW][MAX_D / 128][4];
#pragma unroll
    for (int i = 0; i < RW; ++i)
#pragma unroll
        for (int b = 0; b < MAX_D / 128; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][b][e] = 0.0f;

    for (int kt = walk.start; kt < k_hi; kt = walk.next(kt, TILE)) {
        __syncthreads();                             // the tile before this one has been used
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int e = threadIdx.x + c * (ROWS * 32);
            if (e >= TILE * per_key) continue;
            const int j = e / per_key, w = e - j * per_key;
            float f[PN];
            Piece<T>::unpack(pre[c], f);
            float* dst = w < ck ? Ks + j * ks + w * PN : Vs + j * dv + (w - ck) * PN;
#pragma unroll
            for (int x = 0; x < PN; x += 4)
                *reinterpret_cast<float4*>(dst + x) = make_float4(f[x], f[x + 1], f[x + 2], f[x + 3]);
            if (w == 0) {
                const bool gone = (missing >> c) & 1u;
                Held[j] = gone ? -INFINITY : 0.0f;
                if (gone && status != nullptr) atomicExch(status, 2);
            }
        }
        __syncthreads();
        if (walk.next(kt, TILE) < k_hi) prefetch(walk.next(kt, TILE));   // in flight meanwhile
        if (!any) continue;

        const int kpos = kt + lane;
        const float4* kr = reinterpret_cast<const float4*>(Ks + lane * ks);
        float s[RW];
#pragma unroll
        for (int i = 0; i < RW; ++i) s[i] = 0.0f;
#pragma unroll 4
        for (int d = 0; d < dk / 4; ++d) {
            const float4 kk = kr[d];
#pragma unroll
            for (int i = 0; i < RW; ++i) {
                const float4 qq = reinterpret_cast<const float4*>(Qs + (warp * RW + i) * dk)[d];
                s[i] = fmaf(qq.x, kk.x, s[i]);
                s[i] = fmaf(qq.y, kk.y, s[i]);
                s[i] = fmaf(qq.z, kk.z, s[i]);
                s[i] = fmaf(qq.w, kk.w, s[i]);
            }
        }
        const bool held = Held[lane] == 0.0f;
        float p[RW];
        bool some = false;
#pragma unroll
        for (int i = 0; i < RW; ++i) {
            const bool valid = active[i] && (kpos >= row_lo[i] || kpos < row_first[i]) &&
                               kpos < row_hi[i] && held;
            const float sc = valid ? sight_score(sight, s[i], scale, pen1[i], pen2[i], penalty,
                                                 (float)(pos[i] - kpos))
                                   : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(sc));
            if (m_new == -INFINITY) {               // nothing of this tile is visible to the row
                p[i] = 0.0f;
                continue;
            }
            p[i] = valid ? expf(sc - m_new) : 0.0f;
            const float corr = expf(m[i] - m_new);
            l[i] = l[i] * corr + warp_sum(p[i]);
#pragma unroll
            for (int b = 0; b < MAX_D / 128; ++b)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][b][e] *= corr;
            m[i] = m_new;
            some = true;
        }
        if (!some) continue;
#pragma unroll 4
        for (int j = 0; j < TILE; ++j) {
            float pj[RW];
            bool zero = true;
#pragma unroll
            for (int i = 0; i < RW; ++i) {
                pj[i] = __shfl_sync(0xffffffffu, p[i], j);
                zero &= pj[i] == 0.0f;
            }
            if (zero) continue;                      // the same for the whole warp
#pragma unroll
            for (int b = 0; b < MAX_D / 128; ++b) {
                const int dd = 4 * lane + 128 * b;
                if (dd < dv) {
                    const float4 vv = *reinterpret_cast<const float4*>(Vs + j * dv + dd);
#pragma unroll
                    for (int i = 0; i < RW; ++i) {
                        if (pj[i] == 0.0f) continue;  // as the kernel above skips it
                        acc[i][b][0] = fmaf(pj[i], vv.x, acc[i][b][0]);
                        acc[i][b][1] = fmaf(pj[i], vv.y, acc[i][b][1]);
                        acc[i][b][2] = fmaf(pj[i], vv.z, acc[i][b][2]);
                        acc[i][b][3] = fmaf(pj[i], vv.w, acc[i][b][3]);
                    }
                }
            }
        }
    }
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < RW; ++i) {
        if (!active[i]) continue;
        const float inv = sight_inverse(sight, hq[i], m[i], l[i]);
        const size_t o = (size_t)(tok0 + tok[i]) * out_stride + hq[i] * dv;
#pragma unroll
        for (int b = 0; b < MAX_D / 128; ++b) {
            const int dd = 4 * lane + 128 * b;
            if (dd < dv) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    store_out<T>(out, out_f32, o + dd + e,
                                 acc[i][b][e] * inv * sight_gate<T>(sight, (size_t)(tok0 + tok[i]),
                                                                    hq[i], dv, dd + e));
            }
        }
    }
}


// ------------------------------------------------------------------------------------------
// The same attention for long prompt portions, with the products tiled in registers: a block of
// four warps takes 64 rows, a warp 16 of them against the tile of 32 keys.  Lane (i, j) of a warp
// (i = lane / 8, j = lane % 8) holds rows i, i + 4, i + 8, i + 12 against keys j, j + 8, j + 16,
// j + 24: a step over four features is four 16-byte reads of q and four of k from shared memory
// for 64 multiply-adds (the kernel above: five reads for 16), and rows and keys that meet in one
// read lie 4 banks apart.  The weights go through shared memory once ([key][row], a warp's own
// 2 KB), and for the values lane (i, j) holds the same four rows against columns 4 j + 32 c.
// A row's score sums its features in ascending order, a row's sums over a tile's keys have an
// order of their own (fixed by the key's place in its tile), so a row's result does not depend on
// what shares its tile, its step or its batch.  Sizes as the kernel above.
// ------------------------------------------------------------------------------------------
constexpr int TROWS = 64;

template <typename T, int NC>
__global__ void __launch_bounds__(128, NC <= 4 ? 3 : 2)
attn_chunk_tiled_kernel(const T* __restrict__ q, int q_stride, void* __restrict__ out,
                        int out_stride, const T* __restrict__ k_pages,
                        const T* __restrict__ v_pages, const int* __restrict__ block_table,
                        int table_stride, int num_pages, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                        const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items,
                        const float* __restrict__ r1, const float* __restrict__ r2, int heads,
                        int kv_heads, int dk, int dv, int page, float scale, Sight sight,
                        int out_f32, int* __restrict__ status) {
    constexpr int PN = Piece<T>::N;
    extern __shared__ __align__(16) float smem[];
    const int kst = dk + 4;                          // a key's and a query's stride
    float* Ks = smem;                                // [TILE][kst]
    float* Vs = Ks + TILE * kst;                     // [TILE][dv]
    float* Qs = Vs + TILE * dv;                      // [TROWS][kst]
    float* Ps = Qs + TROWS * kst;                    // [4 warps][TILE][16]
    float* Held = Ps + 4 * TILE * 16;                // [TILE]: 0, or -inf for a key without a page

    const WorkItem it = items[blockIdx.x];
    if (it.kv_begin >= it.kv_end) {
        pdl_wait();
        return;
    }
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int li = lane >> 3, lj = lane & 7;
    const bool penalty = r1 != nullptr;

    bool active[4];
    int tok[4], hq[4], pos[4], row_lo[4], row_hi[4], row_first[4];
    float pen1[4], pen2[4], m[4], l[4];
    bool mine = false;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int r = it.row0 + warp * 16 + li + 4 * e;
        active[e] = r < rows_total;
        mine |= active[e];
        tok[e] = active[e] ? r / g : 0;
        hq[e] = hk * g + (active[e] ? r % g : 0);
        pos[e] = pos0 + tok[e];
        pen1[e] = penalty ? r1[hq[e]] : 0.0f;
        pen2[e] = penalty ? r2[hq[e]] : 0.0f;
        row_lo[e] = max(it.kv_begin, sight_lo(sight, pos[e]));
        row_first[e] = it.kv_begin > 0 ? 0 : sight_first(sight, row_lo[e]);
        row_hi[e] = min(it.kv_end, pos[e] + 1);
        m[e] = -INFINITY;
        l[e] = 0.0f;
    }
    const bool any = __any_sync(0xffffffffu, mine);
    const int last_row = min(it.row0 + TROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    const int k_lo_true = max(it.kv_begin, sight_lo(sight, min_pos));
    const int k_first = it.kv_begin > 0 ? 0 : sight_first(sight, k_lo_true);
    const TileWalk walk(k_lo_true, k_first, TILE);
    const int ck = dk / PN, cv = dv / PN, per_key = ck + cv;

    pdl_wait();
    for (int idx = threadIdx.x; idx < TROWS * dk; idx += 128) {
        const int row = idx / dk, d = idx - row * dk;
        const int r = it.row0 + row;
        float x = 0.0f;
        if (r < rows_total)
            x = to_float(q[(size_t)(tok0 + r / g) * q_stride + (hk * g + r % g) * dk + d]);
        Qs[row * kst + d] = x;
    }

    float acc[4][NC][4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[e][c][x] = 0.0f;

    float* Pw = Ps + warp * TILE * 16;
    for (int kt = walk.start; kt < k_hi; kt = walk.next(kt, TILE)) {
        __syncthreads();                             // the tile before this one has been used
        {
            // four threads a key: thread t takes the key's 16-byte pieces t % 4, t % 4 + 4, ...
            // (keys first, then values), so its key, its page and its row are found once a tile
            const int j = threadIdx.x >> 2, w0 = threadIdx.x & 3;
            const int kpos = kt + j;
            const bool inside = (kpos >= k_lo_true || kpos < k_first) && kpos < k_hi;
            bool gone = false;
            size_t at = 0;
            if (inside) {
                const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
                gone = page_id < 0 || page_id >= num_pages;
                at = ((size_t)page_id * kv_heads + hk) * page + (size_t)(kpos % page);
            }
            const bool read = inside && !gone;
            const T* ksrc = k_pages + at * dk;
            const T* vsrc = v_pages + at * sight.v_stride;
            float* kdst = Ks + j * kst;
            float* vdst = Vs + j * dv;
            for (int w = w0; w < per_key; w += 16) {
                uint4 piece[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {        // four loads in flight a thread
                    const int ww = w + 4 * u;
                    piece[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (read && ww < per_key)
                        piece[u] = *reinterpret_cast<const uint4*>(
                            ww < ck ? ksrc + ww * PN : vsrc + (ww - ck) * PN);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int ww = w + 4 * u;
                    if (ww >= per_key) continue;
                    float f[PN];
                    Piece<T>::unpack(piece[u], f);
                    float* dst = ww < ck ? kdst + ww * PN : vdst + (ww - ck) * PN;
#pragma unroll
                    for (int x = 0; x < PN; x += 4)
                        *reinterpret_cast<float4*>(dst + x) =
                            make_float4(f[x], f[x + 1], f[x + 2], f[x + 3]);
                }
            }
            if (w0 == 0) {
                Held[j] = gone ? -INFINITY : 0.0f;
                if (gone && status != nullptr) atomicExch(status, 2);
            }
        }
        __syncthreads();
        if (!any) continue;

        float s[4][4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[e][c] = 0.0f;
        const float* qb = Qs + (warp * 16 + li) * kst;
        const float* kb = Ks + lj * kst;
#pragma unroll 2
        for (int d = 0; d < dk; d += 4) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) qv[e] = *reinterpret_cast<const float4*>(qb + 4 * e * kst + d);
#pragma unroll
            for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(kb + 8 * c * kst + d);
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[e][c] = fmaf(qv[e].x, kv[c].x, s[e][c]);
                    s[e][c] = fmaf(qv[e].y, kv[c].y, s[e][c]);
                    s[e][c] = fmaf(qv[e].z, kv[c].z, s[e][c]);
                    s[e][c] = fmaf(qv[e].w, kv[c].w, s[e][c]);
                }
        }
        bool held[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) held[c] = Held[lj + 8 * c] == 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float top = -INFINITY;
            bool valid[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int kpos = kt + lj + 8 * c;
                valid[c] = active[e] && (kpos >= row_lo[e] || kpos < row_first[e]) &&
                           kpos < row_hi[e] && held[c];
                s[e][c] = valid[c] ? sight_score(sight, s[e][c], scale, pen1[e], pen2[e], penalty,
                                                 (float)(pos[e] - kpos))
                                   : -INFINITY;
                top = fmaxf(top, s[e][c]);
            }
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 4));
            const float m_new = fmaxf(m[e], top);
            float sum = 0.0f, corr = 1.0f;
            if (m_new == -INFINITY) {                // nothing of this tile is visible to the row
#pragma unroll
                for (int c = 0; c < 4; ++c) s[e][c] = 0.0f;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[e][c] = valid[c] ? expf(s[e][c] - m_new) : 0.0f;
                    sum += s[e][c];
                }
                corr = expf(m[e] - m_new);
                m[e] = m_new;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            l[e] = l[e] * corr + sum;
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[e][c][x] *= corr;
        }
        __syncwarp();                                // the weights of the tile before have been read
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<float4*>(Pw + (lj + 8 * c) * 16 + 4 * li) =
                make_float4(s[0][c], s[1][c], s[2][c], s[3][c]);
        __syncwarp();
        const float* vrow = Vs + 4 * lj;
        const float* prow = Pw + 4 * li;
#pragma unroll 4
        for (int key = 0; key < TILE; ++key, vrow += dv, prow += 16) {
            const float4 pv = *reinterpret_cast<const float4*>(prow);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if (4 * lj + 32 * c < dv) {
                    const float4 vv = *reinterpret_cast<const float4*>(vrow + 32 * c);
                    acc[0][c][0] = fmaf(pv.x, vv.x, acc[0][c][0]); acc[0][c][1] = fmaf(pv.x, vv.y, acc[0][c][1]);
                    acc[0][c][2] = fmaf(pv.x, vv.z, acc[0][c][2]); acc[0][c][3] = fmaf(pv.x, vv.w, acc[0][c][3]);
                    acc[1][c][0] = fmaf(pv.y, vv.x, acc[1][c][0]); acc[1][c][1] = fmaf(pv.y, vv.y, acc[1][c][1]);
                    acc[1][c][2] = fmaf(pv.y, vv.z, acc[1][c][2]); acc[1][c][3] = fmaf(pv.y, vv.w, acc[1][c][3]);
                    acc[2][c][0] = fmaf(pv.z, vv.x, acc[2][c][0]); acc[2][c][1] = fmaf(pv.z, vv.y, acc[2][c][1]);
                    acc[2][c][2] = fmaf(pv.z, vv.z, acc[2][c][2]); acc[2][c][3] = fmaf(pv.z, vv.w, acc[2][c][3]);
                    acc[3][c][0] = fmaf(pv.w, vv.x, acc[3][c][0]); acc[3][c][1] = fmaf(pv.w, vv.y, acc[3][c][1]);
                    acc[3][c][2] = fmaf(pv.w, vv.z, acc[3][c][2]); acc[3][c][3] = fmaf(pv.w, vv.w, acc[3][c][3]);
                }
            }
        }
    }
    pdl_trigger();
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (!active[e]) continue;
        const float inv = sight_inverse(sight, hq[e], m[e], l[e]);
        const size_t o = (size_t)(tok0 + tok[e]) * out_stride + hq[e] * dv;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int col = 4 * lj + 32 * c;
            if (col < dv) {
#pragma unroll
                for (int x = 0; x < 4; ++x)
                    store_out<T>(out, out_f32, o + col + x,
                                 acc[e][c][x] * inv * sight_gate<T>(sight, (size_t)(tok0 + tok[e]),
                                                                    hq[e], dv, col + x));
            }
        }
    }
}


// ------------------------------------------------------------------------------------------
// Steps in which every sequence brings one token.  A block takes a sequence and a kv head; its
// eight warps share the key tiles of the token's chunk out among themselves (warp w takes tiles
// w, w + 8, ...) and each works alone: it asks for its tile's 32 key rows and 32 value rows at
// once (cp.async, 16 bytes a piece, into shared memory of its own), so a tile costs one trip to
// memory; then a lane takes its key's row, and the values come row by row as the weights are
// handed round.  All RW query heads of the group ride on every key read.  The
// warps' partial results (maximum, sum, weighted values) are merged in ascending order of the
// warps.  Sizes as the kernel above; RW >= heads / kv_heads.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}

// What the kernel for single tokens does besides the attention when `on`: it turns its token's
// queries by position (in shared memory), turns and stores the token's key and value of its kv
// head in the pages before it reads them (write_kv; q's row is then [q (H dk) | k (G dk) |
// v (G dv) | ...]), and it finishes every head's result itself - turned back by position where fv
// is given, times sigmoid(gate) where a gate is given, rounded to T - as kv_write_rotated and
// attn_finish_kernel do around the other kernels, with the same arithmetic.
struct Fuse {
    int on;
    const float* fk;
    int rot;
    const float* fv;
    int write_kv;
    const void* gate;
    int ld_gate;
};

template <typename T, int RW>
__global__ void __launch_bounds__(ROWS * 32)
attn_chunk_decode_kernel(const T* __restrict__ q, int q_stride, void* __restrict__ out,
                         int out_stride, T* k_pages, T* v_pages,
                         const int* __restrict__ block_table,
                         int table_stride, int num_pages, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_qstart, const int* __restrict__ seq_pos0,
                         const float* __restrict__ r1, const float* __restrict__ r2, int heads,
                         int kv_heads, int dk, int dv, int page, float scale, Sight sight,
                         int out_f32, Fuse fuse, int* __restrict__ status) {
    constexpr int PN = Piece<T>::N;
    extern __shared__ __align__(16) float smem[];
    float* Qs = smem;                                // [RW][dk]
    float* Pml = Qs + RW * dk;                       // [ROWS warps][RW][2]
    float* Pacc = Pml + ROWS * RW * 2;               // [ROWS warps][RW][dv]
    // a warp's tile: key rows at a stride that keeps 16-byte reads of 8 lanes on different banks
    const int k_stride = ((dk * (int)sizeof(T) + 127) / 128) * 128 + 16;       // bytes
    // values that are the first dv features of the keys (one set of pages, rows of dk) are read
    // from the key tile
    const bool v_in_k = v_pages == k_pages && sight.v_stride == dk;
    const int tile_bytes = TILE * k_stride + (v_in_k ? 0 : TILE * dv * (int)sizeof(T));
    char* mine = reinterpret_cast<char*>(Pacc + ROWS * RW * dv) +
                 (size_t)(threadIdx.x >> 5) * tile_bytes;
    char* Kt = mine;
    const T* Vt = reinterpret_cast<const T*>(mine + TILE * k_stride);
    // a kv head with more than RW query heads is shared by several blocks, RW heads each
    const int parts = gridDim.y / kv_heads;
    const int seq = blockIdx.x, hk = blockIdx.y / parts;
    const int h0 = hk * (heads / kv_heads) + (blockIdx.y % parts) * RW;   // the block's first head
    const int g = min(RW, (hk + 1) * (heads / kv_heads) - h0);            // and how many it has
    const int pos = seq_pos0[seq], slot = seq_slot[seq], tok = seq_qstart[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lo = sight_lo(sight, pos), hi = pos + 1, first = sight_first(sight, lo);
    // the tiles: those of the kept first keys, then from the tile of `lo` on, dealt out in turn
    const TileWalk walk(lo, first, TILE);
    const int first_tiles = walk.jump_at > 0 ? walk.jump_at / TILE : 0;
    const int near0 = walk.jump_at > 0 ? walk.jump_to : walk.start;
    const int n_tiles = first_tiles + (hi - near0 + TILE - 1) / TILE;
    const bool penalty = r1 != nullptr;
    float pen1[RW], pen2[RW], m[RW], l[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) {
        const int hq = h0 + min(i, g - 1);
        pen1[i] = penalty ? r1[hq] : 0.0f;
        pen2[i] = penalty ? r2[hq] : 0.0f;
        m[i] = -INFINITY;
        l[i] = 0.0f;
    }
    pdl_wait();
    for (int e = threadIdx.x; e < RW * dk; e += ROWS * 32) {
        const int i = e / dk, d = e - i * dk;
        Qs[e] = i < g ? to_float(q[(size_t)tok * q_stride + (h0 + i) * dk + d]) : 0.0f;
    }
    __syncthreads();
    if (fuse.on) {
        const float fpos = (float)pos;
        const int half = fuse.rot / 2;
        for (int e = threadIdx.x; e < g * half; e += ROWS * 32) {
            const int i = e / half, p = e - i * half;
            float sn, cs, ra, rb;
            sincosf(fpos * fuse.fk[p], &sn, &cs);
            rope_rotate(Qs[i * dk + p], Qs[i * dk + p + half], cs, sn, ra, rb);
            Qs[i * dk + p] = to_float(from_float<T>(ra));        // rounded as when q goes through memory
            Qs[i * dk + p + half] = to_float(from_float<T>(rb));
        }
        if (fuse.write_kv) {
            const int page_id = block_table[(size_t)slot * table_stride + pos / page];
            if (page_id < 0 || page_id >= num_pages) {           // never written outside the pool
                if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
            } else {
                const size_t at = ((size_t)page_id * kv_heads + hk) * page + (size_t)(pos % page);
                const T* ks = q + (size_t)tok * q_stride + heads * dk + hk * dk;
                const T* vs = q + (size_t)tok * q_stride + (heads + kv_heads) * dk + hk * dv;
                T* kd = k_pages + at * dk;
                T* vd = v_pages + at * dv;
                for (int i = threadIdx.x; i < dk - half; i += ROWS * 32) {
                    if (i < half) {
                        float sn, cs, ra, rb;
                        sincosf(fpos * fuse.fk[i], &sn, &cs);
                        rope_rotate(to_float(ks[i]), to_float(ks[i + half]), cs, sn, ra, rb);
                        kd[i] = from_float<T>(ra);
                        kd[i + half] = from_float<T>(rb);
                    } else {
                        kd[i + half] = ks[i + half];
                    }
                }
                if (fuse.fv != nullptr) {
                    const int vhalf = dv / 2;
                    for (int i = threadIdx.x; i < dv - vhalf; i += ROWS * 32) {
                        if (i < vhalf) {
                            float sn, cs, ra, rb;
                            sincosf(fpos * fuse.fv[i], &sn, &cs);
                            rope_rotate(to_float(vs[i]), to_float(vs[i + vhalf]), cs, sn, ra, rb);
                            vd[i] = from_float<T>(ra);
                            vd[i + vhalf] = from_float<T>(rb);
                        } else {
                            vd[i + vhalf] = vs[i + vhalf];
                        }
                    }
                } else {
                    for (int i = threadIdx.x; i < dv; i += ROWS * 32) vd[i] = vs[i];
                }
            }
        }
        __syncthreads();                             // the block reads what it has just stored
    }
    float acc[RW][MAX_D / 32];
#pragma unroll
    for (int i = 0; i < RW; ++i)
#pragma unroll
        for (int b = 0; b < MAX_D / 32; ++b) acc[i][b] = 0.0f;

    for (int ti = warp; ti < n_tiles; ti += ROWS) {
        const int kt = ti < first_tiles ? ti * TILE : near0 + (ti - first_tiles) * TILE;
        const int kpos = kt + lane;
        bool valid = (kpos >= lo || kpos < first) && kpos < hi;
        size_t row = 0;
        if (valid) {
            const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
            if (page_id < 0 || page_id >= num_pages) {
                valid = false;
                if (status != nullptr) atomicExch(status, 2);
            } else {
                row = ((size_t)page_id * kv_heads + hk) * page + (size_t)(kpos % page);
            }
        }
        __syncwarp();                                // the tile before this one has been used
        {
            const int ck = dk / PN, cv = dv / PN;
            for (int e = lane; e < TILE * ck; e += 32) {
                const int j = e / ck, w = e - j * ck;
                const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, j);
                const bool ok = __shfl_sync(0xffffffffu, (int)valid, j) != 0;
                if (ok) cp_async_16(Kt + j * k_stride + w * 16, k_pages + (size_t)rj * dk + w * PN);
            }
            for (int e = lane; e < (v_in_k ? 0 : TILE * cv); e += 32) {
                const int j = e / cv, w = e - j * cv;
                const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, j);
                const bool ok = __shfl_sync(0xffffffffu, (int)valid, j) != 0;
                if (ok)
                    cp_async_16(mine + TILE * k_stride + ((size_t)j * dv + w * PN) * sizeof(T),
                                v_pages + (size_t)rj * sight.v_stride + w * PN);
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            __syncwarp();
        }
        float s[RW];
#pragma unroll
        for (int i = 0; i < RW; ++i) s[i] = 0.0f;
        const uint4* kp = reinterpret_cast<const uint4*>(Kt + lane * k_stride);
#pragma unroll 4
        for (int piece = 0; piece < dk / PN; ++piece) {
            float f[PN];
            Piece<T>::unpack(valid ? kp[piece] : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
            for (int i = 0; i < RW; ++i) {
                const float4* q4 = reinterpret_cast<const float4*>(Qs + i * dk + piece * PN);
#pragma unroll
                for (int x = 0; x < PN / 4; ++x) {
                    const float4 qq = q4[x];
                    s[i] = fmaf(qq.x, f[4 * x + 0], s[i]);
                    s[i] = fmaf(qq.y, f[4 * x + 1], s[i]);
                    s[i] = fmaf(qq.z, f[4 * x + 2], s[i]);
                    s[i] = fmaf(qq.w, f[4 * x + 3], s[i]);
                }
            }
        }
        float p[RW];
        const float dist = (float)(pos - kpos);
#pragma unroll
        for (int i = 0; i < RW; ++i) {
            const float sc = valid ? sight_score(sight, s[i], scale, pen1[i], pen2[i], penalty, dist)
                                   : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(sc));
            if (m_new == -INFINITY) {
                p[i] = 0.0f;
                continue;
            }
            p[i] = valid ? expf(sc - m_new) : 0.0f;
            const float corr = expf(m[i] - m_new);
            l[i] = l[i] * corr + warp_sum(p[i]);
#pragma unroll
            for (int b = 0; b < MAX_D / 32; ++b) acc[i][b] *= corr;
            m[i] = m_new;
        }
#pragma unroll 4
        for (int j = 0; j < TILE; ++j) {
            float pj[RW];
            bool zero = true;
#pragma unroll
            for (int i = 0; i < RW; ++i) {
                pj[i] = __shfl_sync(0xffffffffu, p[i], j);
                zero &= pj[i] == 0.0f;
            }
            if (zero) continue;
            const T* vr = v_in_k ? reinterpret_cast<const T*>(Kt + j * k_stride) : Vt + (size_t)j * dv;
#pragma unroll
            for (int b = 0; b < MAX_D / 32; ++b) {
                const int dd = lane + 32 * b;
                if (dd < dv) {
                    const float vv = to_float(vr[dd]);
#pragma unroll
                    for (int i = 0; i < RW; ++i) acc[i][b] = fmaf(pj[i], vv, acc[i][b]);
                }
            }
        }
    }
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < RW; ++i) {
        if (lane == 0) {
            Pml[(warp * RW + i) * 2] = m[i];
            Pml[(warp * RW + i) * 2 + 1] = l[i];
        }
#pragma unroll
        for (int b = 0; b < MAX_D / 32; ++b) {
            const int dd = lane + 32 * b;
            if (dd < dv) Pacc[(size_t)(warp * RW + i) * dv + dd] = acc[i][b];
        }
    }
    __syncthreads();
    for (int i = warp; i < g; i += ROWS) {
        float top = -INFINITY;
        for (int w = 0; w < ROWS; ++w) top = fmaxf(top, Pml[(w * RW + i) * 2]);
        float sum = 0.0f, res[MAX_D / 32];
#pragma unroll
        for (int b = 0; b < MAX_D / 32; ++b) res[b] = 0.0f;
        for (int w = 0; w < ROWS; ++w) {
            const float mw = Pml[(w * RW + i) * 2];
            if (mw == -INFINITY) continue;
            const float f = expf(mw - top);
            sum = fmaf(Pml[(w * RW + i) * 2 + 1], f, sum);
#pragma unroll
            for (int b = 0; b < MAX_D / 32; ++b) {
                const int dd = lane + 32 * b;
                if (dd < dv) res[b] = fmaf(Pacc[(size_t)(w * RW + i) * dv + dd], f, res[b]);
            }
        }
        const float inv = sight_inverse(sight, h0 + i, top, sum);
        const size_t o = (size_t)tok * out_stride + (h0 + i) * dv;
        if (fuse.on) {
            // the head's result through shared memory (the place of the first warp's share of
            // this head, which only this warp reads), so that a lane finds its feature's pair
            float* fin = Pacc + (size_t)i * dv;
            __syncwarp();
#pragma unroll
            for (int b = 0; b < MAX_D / 32; ++b) {
                const int dd = lane + 32 * b;
                if (dd < dv) fin[dd] = res[b] * inv;
            }
            __syncwarp();
            const int vhalf = dv / 2;
            const T* gt = fuse.gate
                              ? (const T*)fuse.gate + (size_t)tok * fuse.ld_gate + (h0 + i) * dv
                              : nullptr;
#pragma unroll
            for (int b = 0; b < MAX_D / 32; ++b) {
                const int dd = lane + 32 * b;
                if (dd >= dv) continue;
                float x = fin[dd];
                if (fuse.fv != nullptr && dd < 2 * vhalf) {
                    const int p = dd < vhalf ? dd : dd - vhalf;
                    float sn, cs, ra, rb;
                    sincosf((float)pos * fuse.fv[p], &sn, &cs);
                    rope_rotate(fin[p], fin[p + vhalf], cs, -sn, ra, rb);
                    x = dd < vhalf ? ra : rb;
                }
                if (gt) x *= 1.0f / (1.0f + expf(-to_float(gt[dd])));
                ((T*)out)[o + dd] = from_float<T>(x);
            }
            continue;
        }
#pragma unroll
        for (int b = 0; b < MAX_D / 32; ++b) {
            const int dd = lane + 32 * b;
            if (dd < dv)
                store_out<T>(out, out_f32, o + dd,
                             res[b] * inv * sight_gate<T>(sight, (size_t)tok, h0 + i, dv, dd));
        }
    }
}

}  // namespace

// rows of a tile: 8, or 32 when the step brings prompt portions (`wide`) and the sizes allow the
// kernel that gives a warp four rows
static bool vec_ok(int dtype, int dk, int dv) {
    const int pn = dtype == DE_BF16 ? 8 : 4;
    return dk % pn == 0 && dv % pn == 0 && dk <= MAX_DK && dv <= MAX_D;
}
// the kernel that gives a warp one or four rows holds a tile's 16-byte pieces in at most 16
// registers a thread
static bool vec_fits(int dtype, int dk, int dv) {
    const int pn = dtype == DE_BF16 ? 8 : 4;
    return vec_ok(dtype, dk, dv) && TILE * (dk / pn + dv / pn) <= 16 * ROWS * 32;
}
static size_t tiled_smem(int dk, int dv) {
    return (size_t)(TILE * (dk + 4) + TILE * dv + TROWS * (dk + 4) + 4 * TILE * 16 + TILE) *
           sizeof(float);
}
// `wide`: 0 for steps of single tokens, else the rows (tokens times query heads a kv head) of the
// step's longest portion (1: some portion): from 48 rows on the register-tiled kernel's 64.
DE_EXPORT int de_attn_chunk_rows(int dtype, int dk, int dv, int wide) {
    if (!(vec_ok(dtype, dk, dv) && wide)) return ROWS;
    if (wide >= 48 && tiled_smem(dk, dv) <= 200 * 1024) return TROWS;
    return vec_fits(dtype, dk, dv) ? ROWS * 4 : ROWS;
}

static size_t decode_smem(int dtype, int rw, int dk, int dv, int v_in_k) {
    const int size = dtype == DE_BF16 ? 2 : 4;
    const size_t tile = (size_t)TILE * (((dk * size + 127) / 128) * 128 + 16) +
                        (v_in_k ? 0 : (size_t)TILE * dv * size);
    return (size_t)(rw * dk + ROWS * rw * 2 + ROWS * rw * dv) * sizeof(float) + ROWS * tile;
}

// The query heads a block of the single-token kernel takes (0: the kernel does not take this
// shape).  Keys and values of their own: up to 8 query heads a kv head, all in one block, if the
// eight warps' tiles then fit an SM.  Values inside the keys (`v_in_k`): any number of heads;
// several blocks share a kv head, each with as many heads (up to 8) as fit.
static int decode_rows(int dtype, int heads, int kv_heads, int dk, int dv, int v_in_k) {
    if (!(vec_ok(dtype, dk, dv) && kv_heads > 0 && heads % kv_heads == 0)) return 0;
    const int g = heads / kv_heads;
    int rw = g <= 1 ? 1 : (g <= 2 ? 2 : (g <= 4 ? 4 : 8));
    if (!v_in_k) return g <= 8 && decode_smem(dtype, rw, dk, dv, 0) <= 200 * 1024 ? rw : 0;
    if (decode_smem(dtype, rw, dk, dv, v_in_k) <= 200 * 1024) return rw;
    while ((rw >>= 1) >= 1)
        if (decode_smem(dtype, rw, dk, dv, v_in_k) <= 216 * 1024) return rw;
    return 0;
}

// Whether steps of single tokens go to the kernel that takes a (sequence, kv head) a block, or a
// few blocks where a kv head has many query heads: rows of whole 16-byte pieces, and its eight
// tiles fit an SM.  v_in_k: the values are the first dv features of the keys.
DE_EXPORT int de_attn_chunk_decode_ok(int dtype, int heads, int kv_heads, int dk, int dv,
                                      int v_in_k) {
    return decode_rows(dtype, heads, kv_heads, dk, dv, v_in_k) > 0;
}

DE_EXPORT int de_attn_chunk_decode(int dtype, const void* q, int q_stride, void* out,
                                   int out_stride, void* k_pages, void* v_pages,
                                   const int* block_table, int table_stride, int num_pages,
                                   const int* seq_slot, const int* seq_qstart,
                                   const int* seq_pos0, int n_seqs, const float* r1,
                                   const float* r2, int heads, int kv_heads, int dk, int dv,
                                   int page, float scale, int chunk, int window, int keep_first,
                                   float softcap, int out_f32, int fused, const float* fk, int rot,
                                   const float* fv, int write_kv, const void* gate, int ld_gate,
                                   int v_stride, int linear, const float* sink,
                                   const void* out_gate, int ld_out_gate, int gate_per_head,
                                   int* status, void* stream) {
    if (n_seqs <= 0) return 0;
    // v_stride 0: values in rows of their own; else rows of v_pages are that many elements apart
    const int pn_v = dtype == DE_BF16 ? 8 : 4;
    if (v_stride != 0 && (v_stride < dv || v_stride % pn_v != 0 || fused)) return -2;
    const Sight sight = {chunk, window, keep_first, softcap, v_stride ? v_stride : dv, linear, sink,
                         out_gate, ld_out_gate, gate_per_head};
    if (out_gate != nullptr && fused) return -2;     // a fused step has its own gate
    const Fuse fuse = {fused, fk, rot, fv, write_kv, gate, ld_gate};
    if (fused && (rot < 0 || rot % 2 || rot > dk || (fv != nullptr && dv % 2) || out_f32)) return -2;
    const int v_in_k = v_pages == k_pages && v_stride == dk;
    const int rw = decode_rows(dtype, heads, kv_heads, dk, dv, v_in_k);
    if (rw == 0 || (uintptr_t)k_pages % 16 != 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = heads / kv_heads;
    const size_t smem = decode_smem(dtype, rw, dk, dv, v_in_k);
    if ((uintptr_t)v_pages % 16 != 0) return -2;
    if (g > rw && fused) return -2;         // a kv head's blocks would each store the token's key
    dim3 grid(n_seqs, kv_heads * ((g + rw - 1) / rw));
#define DEC(T, RW)                                                                              \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(attn_chunk_decode_kernel<T, RW>,               \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        return de_launch(attn_chunk_decode_kernel<T, RW>, grid, dim3(ROWS * 32), smem, s,       \
                         (const T*)q, q_stride, out, out_stride, (T*)k_pages, (T*)v_pages,      \
                         block_table, table_stride, num_pages, seq_slot, seq_qstart, seq_pos0,  \
                         r1, r2, heads, kv_heads, dk, dv, page, scale, sight, out_f32, fuse,    \
                         status);                                                               \
    } while (0)
#define DEC_T(T)                                                                                \
    do {                                                                                        \
        if (rw == 1) DEC(T, 1);                                                                 \
        if (rw == 2) DEC(T, 2);                                                                 \
        if (rw == 4) DEC(T, 4);                                                                 \
        DEC(T, 8);                                                                              \
    } while (0)
    if (dtype == DE_BF16) DEC_T(__nv_bfloat16);
    DEC_T(float);
#undef DEC_T
#undef DEC
}

DE_EXPORT int de_kv_write_normed(int dtype, const void* proj, int ld, int k_col,
                                 const int* positions, const int* token_slot, int G, int dk,
                                 int dv, float eps, void* k_pages, void* v_pages,
                                 const int* block_table, int table_stride, int page, int num_pages,
                                 int n, int* status, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 64;
    if (dtype == DE_BF16)
        return de_launch(kv_write_normed_kernel<__nv_bfloat16>, dim3(n, G), dim3(threads), 0, s,
                         (const __nv_bfloat16*)proj, ld, k_col, positions, token_slot, G, dk, dv,
                         eps, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
                         table_stride, page, num_pages, status);
    return de_launch(kv_write_normed_kernel<float>, dim3(n, G), dim3(threads), 0, s,
                     (const float*)proj, ld, k_col, positions, token_slot, G, dk, dv, eps,
                     (float*)k_pages, (float*)v_pages, block_table, table_stride, page, num_pages,
                     status);
}

DE_EXPORT int de_kv_write_rotated(int dtype, void* proj, int ld, const int* positions,
                                  const int* token_slot, const float* fk, int rot, const float* fv,
                                  int H, int G, int dk, int dv, void* k_pages, void* v_pages,
                                  const int* block_table, int table_stride, int page,
                                  int num_pages, int write_kv, int n, int* status, void* stream) {
    if (n <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > dk || (fv != nullptr && dv % 2)) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int work = (H + G) * dk + G * dv;
    const int threads = n >= 512 ? 128 : (work >= 2048 ? 512 : 256);
    if (dtype == DE_BF16)
        return de_launch(kv_write_rotated_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s,
                         (__nv_bfloat16*)proj, ld, positions, token_slot, fk, rot, fv, H, G, dk, dv,
                         (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
                         table_stride, page, num_pages, write_kv, status);
    return de_launch(kv_write_rotated_kernel<float>, dim3(n), dim3(threads), 0, s, (float*)proj, ld,
                     positions, token_slot, fk, rot, fv, H, G, dk, dv, (float*)k_pages,
                     (float*)v_pages, block_table, table_stride, page, num_pages, write_kv, status);
}

DE_EXPORT int de_qkv_prepare(int dtype, const void* proj, int ld, void* q_out,
                             const int* positions, const int* token_seq, const int* token_slot,
                             const int* seq_pos0, const float* bias, const float* taps, int K,
                             float* state, long long slot_stride, int conv_offset, int norm,
                             const float* q_weight, const float* k_weight, float eps,
                             const float* freq, int rot, float magnitude, int adjacent,
                             float temp_coef, int temp_every, int mix, const float* lambda,
                             float* v_first, int keep_here, int H, int G, int dk, int dv,
                             void* k_pages, void* v_pages, const int* block_table,
                             int table_stride, int page, int num_pages, int n, int* status,
                             void* stream) {
    if (n <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > dk || (rot > 0 && freq == nullptr) || norm < 0 || norm > 2 ||
        (norm != 0 && (q_weight == nullptr || k_weight == nullptr)) || mix < 0 || mix > 2 ||
        (mix != 0 && v_first == nullptr) || (mix == 2 && lambda == nullptr) ||
        (taps != nullptr && (K < 1 || (K > 1 && state == nullptr))))
        return -2;
    const Prepare pp = {bias, taps, K, state, slot_stride, conv_offset, norm, q_weight, k_weight,
                        eps, freq, rot, magnitude, adjacent, temp_coef, temp_every, mix, lambda,
                        v_first, keep_here};
    cudaStream_t s = (cudaStream_t)stream;
    const int C = (H + G) * dk + G * dv;
    const size_t smem = (size_t)(C + rot + H + G) * sizeof(float);
    if (smem > 200 * 1024) return -2;
    const int threads = C >= 2048 && n < 512 ? 512 : 256;
    const int pn = dtype == DE_BF16 ? 8 : 4;
    const bool vec = C % pn == 0 && ld % pn == 0 && (uintptr_t)proj % 16 == 0;
#define PREP(T, V)                                                                              \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            cudaError_t e = cudaFuncSetAttribute(qkv_prepare_kernel<T, V>,                      \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                                 (int)smem);                                    \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        return de_launch(qkv_prepare_kernel<T, V>, dim3(n), dim3(threads), smem, s,             \
                         (const T*)proj, ld, (T*)q_out, positions, token_seq, token_slot,       \
                         seq_pos0, pp, H, G, dk, dv, (T*)k_pages, (T*)v_pages, block_table,     \
                         table_stride, page, num_pages, status);                                \
    } while (0)
    if (dtype == DE_BF16) {
        if (vec) PREP(__nv_bfloat16, true);
        PREP(__nv_bfloat16, false);
    }
    if (vec) PREP(float, true);
    PREP(float, false);
#undef PREP
}

DE_EXPORT int de_conv_keep(int dtype, const void* proj, int ld, float* state, long long slot_stride,
                           int conv_offset, const int* seq_slot, const int* seq_qstart,
                           const int* seq_qlen, int n_seqs, int C, int K, void* stream) {
    if (n_seqs <= 0 || K <= 1) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DE_BF16)
        return de_launch(conv_keep_kernel<__nv_bfloat16>, dim3(n_seqs), dim3(256), 0, s,
                         (const __nv_bfloat16*)proj, ld, state, slot_stride, conv_offset, seq_slot,
                         seq_qstart, seq_qlen, C, K);
    return de_launch(conv_keep_kernel<float>, dim3(n_seqs), dim3(256), 0, s, (const float*)proj,
                     ld, state, slot_stride, conv_offset, seq_slot, seq_qstart, seq_qlen, C, K);
}

DE_EXPORT int de_attn_finish(int dtype, const float* o, const int* positions, const float* fv,
                             const void* gate, int ld_gate, void* out, int n, int H, int dv,
                             int gate_per_head, void* stream) {
    if (n <= 0) return 0;
    if (fv != nullptr && dv % 2) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = n >= 512 ? 128 : (H * dv >= 2048 ? 512 : 256);
    if (dtype == DE_BF16)
        return de_launch(attn_finish_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s, o,
                         positions, fv, (const __nv_bfloat16*)gate, ld_gate, (__nv_bfloat16*)out, H,
                         dv, gate_per_head);
    return de_launch(attn_finish_kernel<float>, dim3(n), dim3(threads), 0, s, o, positions, fv,
                     (const float*)gate, ld_gate, (float*)out, H, dv, gate_per_head);
}

DE_EXPORT int de_attn_chunk(int dtype, const void* q, int q_stride, void* out, int out_stride,
                            const void* k_pages, const void* v_pages, const int* block_table,
                            int table_stride, int num_pages, const int* seq_slot,
                            const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                            const int* items, int num_items, const float* r1, const float* r2,
                            int heads, int kv_heads, int dk, int dv, int page, float scale,
                            int chunk, int window, int keep_first, float softcap, int out_f32,
                            int tile_rows, int v_stride, int linear, const float* sink,
                            const void* out_gate, int ld_out_gate, int gate_per_head,
                            int* status, void* stream) {
    if (num_items <= 0) return 0;
    // v_stride 0: values in rows of their own; else rows of v_pages are that many elements apart
    if (v_stride != 0 && (v_stride < dv || (vec_ok(dtype, dk, dv) && v_stride % (dtype == DE_BF16 ? 8 : 4))))
        return -2;
    const Sight sight = {chunk, window, keep_first, softcap, v_stride ? v_stride : dv, linear, sink,
                         out_gate, ld_out_gate, gate_per_head};
    if (dk <= 0 || dk > MAX_DK || dv <= 0 || dv > MAX_D || heads % kv_heads != 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    if (tile_rows != ROWS && !((tile_rows == ROWS * 4 && vec_fits(dtype, dk, dv)) ||
                               (tile_rows == TROWS && vec_ok(dtype, dk, dv))))
        return -5;
    if (tile_rows == TROWS) {
        if ((uintptr_t)k_pages % 16 != 0 || (uintptr_t)v_pages % 16 != 0) return -5;
        const size_t tsmem = tiled_smem(dk, dv);
        if (tsmem > 200 * 1024) return -5;
        const int nc = (dv + 31) / 32;
        dim3 tgrid(num_items, kv_heads);
#define TILED(T, NC)                                                                            \
    do {                                                                                        \
        if (tsmem > 48 * 1024) {                                                                \
            cudaError_t te = cudaFuncSetAttribute(attn_chunk_tiled_kernel<T, NC>,               \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                  (int)tsmem);                                  \
            if (te != cudaSuccess) return (int)te;                                              \
        }                                                                                       \
        return de_launch(attn_chunk_tiled_kernel<T, NC>, tgrid, dim3(128), tsmem, s,            \
                         (const T*)q, q_stride, out, out_stride, (const T*)k_pages,             \
                         (const T*)v_pages, block_table, table_stride, num_pages, seq_slot,     \
                         seq_qstart, seq_qlen, seq_pos0, (const WorkItem*)items, r1, r2, heads, \
                         kv_heads, dk, dv, page, scale, sight, out_f32, status);                \
    } while (0)
#define TILED_N(T)                                                                              \
    do {                                                                                        \
        if (nc <= 1) TILED(T, 1);                                                               \
        if (nc <= 2) TILED(T, 2);                                                               \
        if (nc <= 4) TILED(T, 4);                                                               \
        TILED(T, 8);                                                                            \
    } while (0)
        if (dtype == DE_BF16) TILED_N(__nv_bfloat16);
        TILED_N(float);
#undef TILED_N
#undef TILED
    }
    if (vec_fits(dtype, dk, dv) && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0) {
        const int rw = tile_rows / ROWS;
        const int pn = dtype == DE_BF16 ? 8 : 4;
        const int pieces = TILE * (dk / pn + dv / pn);
        const int nch = (pieces + ROWS * 32 - 1) / (ROWS * 32);
        const size_t vsmem = (size_t)(TILE * (((dk + 31) / 32) * 32 + 4) + TILE * dv +
                                      ROWS * rw * dk + TILE) * sizeof(float);
        dim3 vgrid(num_items, kv_heads);
#define VEC(T, RW, NCH)                                                                         \
    do {                                                                                        \
        if (vsmem > 48 * 1024) {                                                                \
            cudaError_t ve = cudaFuncSetAttribute(attn_chunk_vec_kernel<T, RW, NCH>,            \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                  (int)vsmem);                                  \
            if (ve != cudaSuccess) return (int)ve;                                              \
        }                                                                                       \
        return de_launch(attn_chunk_vec_kernel<T, RW, NCH>, vgrid, dim3(ROWS * 32), vsmem, s,   \
                         (const T*)q, q_stride, out, out_stride, (const T*)k_pages,             \
                         (const T*)v_pages, block_table, table_stride, num_pages, seq_slot,     \
                         seq_qstart, seq_qlen, seq_pos0, (const WorkItem*)items, r1, r2, heads, \
                         kv_heads, dk, dv, page, scale, sight, out_f32, status);                \
    } while (0)
#define VEC_N(T, RW)                                                                            \
    do {                                                                                        \
        if (nch <= 2) VEC(T, RW, 2);                                                            \
        if (nch <= 4) VEC(T, RW, 4);                                                            \
        if (nch <= 8) VEC(T, RW, 8);                                                            \
        VEC(T, RW, 16);                                                                         \
    } while (0)
        if (dtype == DE_BF16) {
            if (rw == 4) VEC_N(__nv_bfloat16, 4);
            VEC_N(__nv_bfloat16, 1);
        }
        if (rw == 4) VEC_N(float, 4);
        VEC_N(float, 1);
#undef VEC_N
#undef VEC
    }
    const size_t smem = (size_t)(TILE * (dk + 1) + TILE * dv + ROWS * dk) * sizeof(float);
    dim3 grid(num_items, kv_heads);
    cudaError_t e;
#define LAUNCH(T)                                                                               \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            e = cudaFuncSetAttribute(attn_chunk_kernel<T>,                                      \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        return de_launch(attn_chunk_kernel<T>, grid, dim3(ROWS * 32), smem, s, (const T*)q,     \
                         q_stride, out, out_stride, (const T*)k_pages, (const T*)v_pages,       \
                         block_table, table_stride, num_pages, seq_slot, seq_qstart, seq_qlen,  \
                         seq_pos0, (const WorkItem*)items, r1, r2, heads, kv_heads, dk, dv, page, \
                         scale, sight, out_f32, status);                                        \
    } while (0)
    if (dtype == DE_BF16) LAUNCH(__nv_bfloat16);
    LAUNCH(float);
#undef LAUNCH
}
