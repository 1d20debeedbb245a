// A routed feed-forward: every token runs `top` of `experts` small gated feed-forwards.
//
// mx_moe_route: per token the router's logits z = R h on the FP32 cores (R float [experts][K]), scores
//   s = sigmoid(z), and the choice: the experts form `n_groups` runs of neighbours, a run is worth the sum of its
//   two largest scores, only the `keep` best runs may supply experts, and of those the `top` largest scores win
//   (ties go to the lower index). The weights are the winners' scores over their sum (+ 1e-20) times `scale`.
//   The kernel also counts the pairs of every expert and gives each (token, slot) pair its place among its
//   expert's pairs (the order inside an expert is whatever the atomics make it: every row of a grouped product
//   depends on that row alone, so the order changes no number).
// mx_moe_route_softmax: the same outputs from another rule. The router has `n_experts + n_identity` rows; the scores
//   are the softmax over all of them (of logit + bias[e] where a bias is given: with it and no correction the rule is
//   "the `top` largest logits, weighted by the softmax over those alone"); the choice ranks score + correction[e] (a float per row, optional) and takes the
//   `top` largest (ties to the lower index); the weights are the winners' plain scores over their sum (+ 1e-20). The
//   last `n_identity` rows stand for experts without matrices that return their input: such a pair keeps its id
//   (>= n_experts), is counted nowhere and gets no sorted row; the combine kernels add weight * input for it.
// mx_moe_plan (one block): from the counts, the first sorted row of every expert and the list of row tiles
//   (expert, first sorted row, rows) that the grouped products walk; the number of tiles stays on the device.
// mx_moe_scatter: order[first[e] + place] = pair: the pairs sorted by expert.
// mx_moe_gemm: the grouped product over the sorted rows, a block per (row tile, column tile), on the FP32 cores
//   with float accumulators (operands float or bfloat16). GLU form: rows gathered from the tokens' activations,
//   two accumulators (gate rows and up rows of the expert's stacked matrix), out = act(gate) * up in the operand
//   type. Plain form: rows are the sorted rows themselves, out[pair] = weight[pair] * product in float, one row per
//   pair, so that the sum over a token's pairs can be formed in a fixed order.
// mx_moe_combine: residual[t] += sum over the token's pairs, slot 0 first.
// mx_moe_gather, mx_moe_combine_sorted: the ends of the tensor-core path. The grouped tcgen05 product
//   (mx_gemm_tcgen05_grouped) reads its rows through TMA, so the tokens' rows are first copied into the order of
//   the sorted pairs; it writes rows in that order too, and the combine step finds a pair's row at
//   first[expert] + place and weighs it there. The plan's tiles are 128 rows then (32 for the FP32-core product).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MOE_BM = 32, MOE_BN = 64, MOE_BK = 16;

__device__ __forceinline__ void arg_best(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
    }
}

// z[e] = router[e] . h for every router row, in float: the token's activations staged in shared memory (h_s [K]),
// a warp per row. Ends with a barrier: every thread may read z afterwards.
template <typename T>
__device__ __forceinline__ void router_logits(const T* __restrict__ h, const float* __restrict__ router, int K,
                                              int n_rows, float* h_s, float* z_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int k = tid; k < K; k += blockDim.x) h_s[k] = to_float(h[k]);
    __syncthreads();
    const bool vec = K % 4 == 0 && (reinterpret_cast<uintptr_t>(router) & 15) == 0;
    for (int e = warp; e < n_rows; e += blockDim.x >> 5) {
        const float* w = router + (size_t)e * K;
        float z = 0.f;
        if (vec) {
            // four 16-byte loads of a lane set out together: a row of 2,048 costs four trips to memory, not 64
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* h4 = reinterpret_cast<const float4*>(h_s);
            const int k4 = K >> 2;
            float zz[4] = {0.f, 0.f, 0.f, 0.f};
            for (int k = lane; k < k4; k += 128) {
                float4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    wv[u] = (k + 32 * u < k4) ? w4[k + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (k + 32 * u < k4) {
                        const float4 hv = h4[k + 32 * u];
                        zz[u] = fmaf(wv[u].x, hv.x, zz[u]);
                        zz[u] = fmaf(wv[u].y, hv.y, zz[u]);
                        zz[u] = fmaf(wv[u].z, hv.z, zz[u]);
                        zz[u] = fmaf(wv[u].w, hv.w, zz[u]);
                    }
                }
            }
            z = (zz[0] + zz[1]) + (zz[2] + zz[3]);
        } else {
            for (int k = lane; k < K; k += 32) z = fmaf(w[k], h_s[k], z);
        }
        z = warp_sum(z);
        if (lane == 0) z_out[e] = z;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, int ld, const float* __restrict__ router, int K, int n_experts, int top,
                 int n_groups, int keep, float scale, int* __restrict__ ids, float* __restrict__ weights,
                 int* __restrict__ counts, int* __restrict__ place) {
    extern __shared__ __align__(16) float route_s[];
    float* h_s = route_s;                         // [K]
    float* score = h_s + K;                       // [experts]
    float* open = score + n_experts;              // [experts]: the score while the expert may still be chosen, else -1
    float* worth = open + n_experts;              // [groups]
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    router_logits(h + (size_t)t * ld, router, K, n_experts, h_s, score);
    for (int e = tid; e < n_experts; e += blockDim.x) score[e] = 1.0f / (1.0f + expf(-score[e]));
    __syncthreads();
    if (warp != 0) return;
    const int per = n_experts / n_groups;
    const bool limited = n_groups > 1 && keep < n_groups;
    for (int g = lane; g < n_groups; g += 32) {
        float a = -1.f, b = -1.f;                 // the two largest of the run (scores are positive)
        for (int e = g * per; e < (g + 1) * per; ++e) {
            const float s = score[e];
            if (s > a) { b = a; a = s; } else if (s > b) { b = s; }
        }
        worth[g] = a + (per > 1 ? b : 0.f);
    }
    for (int e = lane; e < n_experts; e += 32) open[e] = limited ? -1.f : score[e];
    __syncwarp();
    if (limited) {
        for (int round = 0; round < keep; ++round) {
            float v = -2.f;
            int i = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32)
                if (worth[g] > v) { v = worth[g]; i = g; }
            arg_best(v, i);
            __syncwarp();
            if (lane == 0) worth[i] = -3.f;
            for (int e = i * per + lane; e < (i + 1) * per; e += 32) open[e] = score[e];
            __syncwarp();
        }
    }
    float total = 0.f, mine = 0.f;
    int my_id = 0;
    for (int slot = 0; slot < top; ++slot) {
        float v = -2.f;
        int i = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32)
            if (open[e] > v) { v = open[e]; i = e; }
        arg_best(v, i);
        __syncwarp();
        if (lane == 0) open[i] = -3.f;
        __syncwarp();
        total += v;
        if (lane == slot % 32 && slot / 32 == 0) { mine = v; my_id = i; }
        if (slot >= 32 && lane == 0) {            // more slots than lanes: written one by one
            ids[(size_t)t * top + slot] = i;
            weights[(size_t)t * top + slot] = v;  // normalised below
            place[(size_t)t * top + slot] = atomicAdd(&counts[i], 1);
        }
    }
    const float norm = scale / (total + 1e-20f);
    if (lane < min(top, 32)) {
        ids[(size_t)t * top + lane] = my_id;
        weights[(size_t)t * top + lane] = mine * norm;
        place[(size_t)t * top + lane] = atomicAdd(&counts[my_id], 1);
    }
    __syncwarp();
    if (lane == 0)
        for (int slot = 32; slot < top; ++slot) weights[(size_t)t * top + slot] *= norm;
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_softmax_kernel(const T* __restrict__ h, int ld, const float* __restrict__ router, int K, int n_experts,
                         int n_identity, int top, const float* __restrict__ correction,
                         const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
                         int* __restrict__ counts, int* __restrict__ place) {
    extern __shared__ __align__(16) float route_s[];
    const int n_rows = n_experts + n_identity;
    float* h_s = route_s;                         // [K]
    float* score = h_s + K;                       // [rows]: logits, then softmax scores
    float* open = score + n_rows;                 // [rows]: score + correction while the row may still be chosen
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    router_logits(h + (size_t)t * ld, router, K, n_rows, h_s, score);
    if (threadIdx.x >= 32) return;
    float m = -INFINITY;
    for (int e = lane; e < n_rows; e += 32) {
        if (bias) score[e] += bias[e];           // part of the logit: it moves scores, choice and weights alike
        m = fmaxf(m, score[e]);
    }
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < n_rows; e += 32) {
        const float v = expf(score[e] - m);
        score[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < n_rows; e += 32) {
        const float sc = score[e] / sum;
        score[e] = sc;
        open[e] = sc + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    float total = 0.f;
    for (int slot = 0; slot < top; ++slot) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int e = lane; e < n_rows; e += 32)
            if (open[e] > v) { v = open[e]; i = e; }
        arg_best(v, i);
        if (i >= n_rows) i = 0;                   // nothing comparable left (scores that are no numbers)
        __syncwarp();
        const float sc = score[i];
        if (lane == 0) {
            open[i] = -INFINITY;
            ids[(size_t)t * top + slot] = i;
            weights[(size_t)t * top + slot] = sc;  // normalised below
            place[(size_t)t * top + slot] = i < n_experts ? atomicAdd(&counts[i], 1) : 0;
        }
        __syncwarp();
        total += sc;
    }
    const float norm = 1.f / (total + 1e-20f);
    __syncwarp();
    for (int slot = lane; slot < top; slot += 32) weights[(size_t)t * top + slot] *= norm;
}

__global__ void moe_plan_kernel(const int* __restrict__ counts, int n_experts, int tile_rows, int* __restrict__ first,
                                int* __restrict__ tile_map, int* __restrict__ n_tiles) {
    extern __shared__ int plan_s[];               // [experts + 1]: first tile of every expert
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = rows;
            plan_s[e] = tiles;
            rows += counts[e];
            tiles += (counts[e] + tile_rows - 1) / tile_rows;
        }
        first[n_experts] = rows;
        plan_s[n_experts] = tiles;
        n_tiles[0] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int count = counts[e], row0 = first[e];
        for (int i = 0, tile = plan_s[e]; i * tile_rows < count; ++i, ++tile) {
            tile_map[3 * tile] = e;
            tile_map[3 * tile + 1] = row0 + i * tile_rows;
            tile_map[3 * tile + 2] = min(tile_rows, count - i * tile_rows);
        }
    }
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ place,
                                   const int* __restrict__ first, int* __restrict__ order, int n_pairs,
                                   int n_experts) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    // a pair of an expert without matrices (id >= n_experts) has no sorted row
    if (p < n_pairs && ids[p] < n_experts) order[first[ids[p]] + place[p]] = p;
}

__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + expf(-g)); }

// the gate capped from above, the linear branch from both sides (limit <= 0: neither), a sigmoid of a slope, a shift
struct ClampedAct { float limit, slope, shift; };
__device__ __forceinline__ float act_clamped(float g, float u, const ClampedAct& c) {
    if (c.limit > 0.f) {
        g = fminf(g, c.limit);
        u = fminf(fmaxf(u, -c.limit), c.limit);
    }
    return g / (1.0f + expf(-c.slope * g)) * (u + c.shift);
}

// ACT: 0 = gelu (tanh form), 1 = silu, 2 = clamped (ClampedAct)
template <typename T, bool GLU, int ACT>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, int lda, const int* __restrict__ order, int a_div, const T* __restrict__ w,
                long long expert_stride, int N, int K, const int* __restrict__ tile_map,
                const int* __restrict__ n_tiles, void* __restrict__ out_raw, const float* __restrict__ pair_weight,
                const ClampedAct clamped) {
    if ((int)blockIdx.y >= n_tiles[0]) return;
    __shared__ float a_s[MOE_BK][MOE_BM + 1], w_s[MOE_BK][MOE_BN + 1], u_s[GLU ? MOE_BK : 1][MOE_BN + 1];
    __shared__ int src_row[MOE_BM];
    const int expert = tile_map[3 * blockIdx.y], row0 = tile_map[3 * blockIdx.y + 1], rows = tile_map[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_BN, tid = threadIdx.x;
    if (tid < MOE_BM) src_row[tid] = tid < rows ? (GLU ? order[row0 + tid] / a_div : row0 + tid) : -1;
    __syncthreads();
    const T* we = w + (size_t)expert * expert_stride;
    const int tx = tid & 15, ty = tid >> 4;                   // 4 columns, 2 rows a thread
    float acc[2][4] = {}, acc_u[2][4] = {};
    const int a_row = tid >> 3, a_k = (tid & 7) * 2;          // this thread's two elements of the row tile
    const int w_row = tid >> 2, w_k = (tid & 3) * 4;          // ... and four of each weight tile
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        {
            const int r = src_row[a_row];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int k = k0 + a_k + e;
                a_s[a_k + e][a_row] = (r >= 0 && k < K) ? to_float(a[(size_t)r * lda + k]) : 0.f;
            }
            const int n = n0 + w_row;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = k0 + w_k + e;
                const bool ok = n < N && k < K;
                w_s[w_k + e][w_row] = ok ? to_float(we[(size_t)n * K + k]) : 0.f;
                if (GLU) u_s[w_k + e][w_row] = ok ? to_float(we[(size_t)(N + n) * K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MOE_BK; ++k) {
            const float a0 = a_s[k][2 * ty], a1 = a_s[k][2 * ty + 1];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float wv = w_s[k][4 * tx + c];
                acc[0][c] = fmaf(a0, wv, acc[0][c]);
                acc[1][c] = fmaf(a1, wv, acc[1][c]);
                if (GLU) {
                    const float uv = u_s[k][4 * tx + c];
                    acc_u[0][c] = fmaf(a0, uv, acc_u[0][c]);
                    acc_u[1][c] = fmaf(a1, uv, acc_u[1][c]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = 2 * ty + r;
        if (row >= rows) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = n0 + 4 * tx + c;
            if (n >= N) continue;
            if (GLU) {
                const float g = acc[r][c];
                const float value = ACT == 2 ? act_clamped(g, acc_u[r][c], clamped)
                                             : (ACT == 0 ? gelu_tanh(g) : act_silu(g)) * acc_u[r][c];
                reinterpret_cast<T*>(out_raw)[(size_t)(row0 + row) * N + n] = from_float<T>(value);
            } else {
                const int pair = order[row0 + row];
                reinterpret_cast<float*>(out_raw)[(size_t)pair * N + n] = acc[r][c] * pair_weight[pair];
            }
        }
    }
}

// `ids` / `input` (both or neither): a pair whose id is >= n_experts belongs to an expert that returns its input;
// nobody wrote its row, and weight[pair] * input[t] stands for it (input in float or bfloat16)
template <typename TIn>
__global__ void moe_combine_kernel(const float* __restrict__ pairs, float* __restrict__ residual, int top, int width,
                                   long long count, const int* __restrict__ ids, const float* __restrict__ weight,
                                   const TIn* __restrict__ input, int input_ld, int n_experts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    float sum = 0.f;
    for (int s = 0; s < top; ++s) {
        const long long pair = t * top + s;
        if (ids && ids[pair] >= n_experts) sum += weight[pair] * to_float(input[(size_t)t * input_ld + c]);
        else sum += pairs[(size_t)pair * width + c];
    }
    residual[i] += sum;
}

// rows of the tokens' activations in the order of the sorted pairs: what a TMA-fed grouped product reads
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ h, int ld, const int* __restrict__ order, int top,
                                  __nv_bfloat16* __restrict__ sorted, int K8, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long r = i / K8;
    const int c = (int)(i - r * K8);
    const int token = order[r] / top;
    reinterpret_cast<uint4*>(sorted)[i] = *reinterpret_cast<const uint4*>(h + (size_t)token * ld + 8 * c);
}

// residual[t] += sum over the token's pairs of weight[pair] * rows[place of the pair among the sorted rows]
template <typename TIn>
__global__ void moe_combine_sorted_kernel(const float* __restrict__ rows, const int* __restrict__ ids,
                                          const int* __restrict__ place, const int* __restrict__ first,
                                          const float* __restrict__ weight, float* __restrict__ residual, int top,
                                          int width, long long count, const TIn* __restrict__ input, int input_ld,
                                          int n_experts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    float sum = 0.f;
    for (int s = 0; s < top; ++s) {
        const long long pair = t * top + s;
        const int e = ids[pair];
        if (e >= n_experts) sum += weight[pair] * to_float(input[(size_t)t * input_ld + c]);
        else sum += weight[pair] * rows[((size_t)first[e] + place[pair]) * width + c];
    }
    residual[i] += sum;
}

// the same, four columns a thread (width a multiple of 4, 16-byte aligned rows)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename TIn>
__global__ void moe_combine_sorted_vec_kernel(const float* __restrict__ rows, const int* __restrict__ ids,
                                              const int* __restrict__ place, const int* __restrict__ first,
                                              const float* __restrict__ weight, float* __restrict__ residual, int top,
                                              int width4, long long count, const TIn* __restrict__ input,
                                              int input_ld, int n_experts) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long t = i / width4;
    const int c = (int)(i - t * width4);
    float4 sum = reinterpret_cast<const float4*>(residual)[i];
    for (int s = 0; s < top; ++s) {
        const long long pair = t * top + s;
        const float w = weight[pair];
        const int e = ids[pair];
        const float4 v = e >= n_experts ? load4(input + (size_t)t * input_ld + 4 * (size_t)c)
                                        : reinterpret_cast<const float4*>(rows)[((size_t)first[e] + place[pair]) * width4 + c];
        sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
    }
    reinterpret_cast<float4*>(residual)[i] = sum;
}

template <typename T>
__global__ void glu_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int ff, int act, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long t = i / ff;
    const int c = (int)(i - t * ff);
    const float g = to_float(gu[(size_t)t * ld + c]);
    const float u = to_float(gu[(size_t)t * ld + ff + c]);
    out[i] = from_float<T>((act == 0 ? gelu_tanh(g) : act_silu(g)) * u);
}

// eight neighbouring columns a thread, 16-byte accesses (bfloat16 rows whose width and stride are multiples of 8)
__global__ void glu_vec_kernel(const __nv_bfloat16* __restrict__ gu, int ld, __nv_bfloat16* __restrict__ out, int ff,
                               int act, long long groups) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = ff >> 3;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) << 3;
    const uint4 graw = *reinterpret_cast<const uint4*>(gu + (size_t)t * ld + c);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gu + (size_t)t * ld + ff + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float g0 = __low2float(g2[e]), g1 = __high2float(g2[e]);
        const float a0 = act == 0 ? gelu_tanh(g0) : act_silu(g0), a1 = act == 0 ? gelu_tanh(g1) : act_silu(g1);
        o2[e] = __floats2bfloat162_rn(a0 * __low2float(u2[e]), a1 * __high2float(u2[e]));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ff + c) = oraw;
}

}  // namespace

extern "C" int mx_moe_route(const void* h, int dtype, int ld, const float* router, int K, int n_experts, int top,
                            int n_groups, int keep, float scale, int* ids, float* weights, int* counts, int* place,
                            int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (n_experts <= 0 || top <= 0 || top > n_experts) MX_REFUSE("router: top %d of %d experts", top, n_experts);
    if (n_groups <= 0 || n_experts % n_groups != 0) MX_REFUSE("router: %d experts in %d equal groups", n_experts, n_groups);
    if (keep <= 0 || keep > n_groups) MX_REFUSE("router: %d of %d groups kept", keep, n_groups);
    if (keep * (n_experts / n_groups) < top) MX_REFUSE("router: %d kept groups hold fewer than %d experts", keep, top);
    const size_t smem = ((size_t)K + 2 * (size_t)n_experts + n_groups) * sizeof(float);
    if (smem > 48 * 1024) MX_REFUSE("router: %zu bytes of shared memory for K = %d and %d experts", smem, K, n_experts);
    if (dtype == MX_DTYPE_F32)
        moe_route_kernel<float><<<n_tokens, 256, smem, stream>>>((const float*)h, ld, router, K, n_experts, top, n_groups,
                                                                keep, scale, ids, weights, counts, place);
    else
        moe_route_kernel<__nv_bfloat16><<<n_tokens, 256, smem, stream>>>((const __nv_bfloat16*)h, ld, router, K, n_experts,
                                                                        top, n_groups, keep, scale, ids, weights, counts,
                                                                        place);
    return mx_launch_status();
}

extern "C" int mx_moe_route_softmax(const void* h, int dtype, int ld, const float* router, int K, int n_experts,
                                    int n_identity, int top, const float* correction, const float* bias, int* ids,
                                    float* weights, int* counts, int* place, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    const int n_rows = n_experts + n_identity;
    if (n_experts < 0 || n_identity < 0 || top <= 0 || top > n_rows)
        MX_REFUSE("router: top %d of %d experts and %d without matrices", top, n_experts, n_identity);
    const size_t smem = ((size_t)K + 2 * (size_t)n_rows) * sizeof(float);
    if (smem > 48 * 1024) MX_REFUSE("router: %zu bytes of shared memory for K = %d and %d rows", smem, K, n_rows);
    if (dtype == MX_DTYPE_F32)
        moe_route_softmax_kernel<float><<<n_tokens, 256, smem, stream>>>((const float*)h, ld, router, K, n_experts,
                                                                        n_identity, top, correction, bias, ids,
                                                                        weights, counts, place);
    else
        moe_route_softmax_kernel<__nv_bfloat16><<<n_tokens, 256, smem, stream>>>(
            (const __nv_bfloat16*)h, ld, router, K, n_experts, n_identity, top, correction, bias, ids, weights, counts,
            place);
    return mx_launch_status();
}

extern "C" int mx_moe_tile_rows() { return MOE_BM; }

extern "C" int mx_moe_plan(const int* counts, const int* ids, const int* place, int n_experts, int n_pairs, int tile_rows,
                           int* first, int* tile_map, int* n_tiles, int* order, cudaStream_t stream) {
    if (n_pairs <= 0) return MX_OK;
    if (n_experts > 8192) MX_REFUSE("routed feed-forward: %d experts", n_experts);
    if (tile_rows <= 0) MX_REFUSE("routed feed-forward: row tiles of %d rows", tile_rows);
    moe_plan_kernel<<<1, 256, (size_t)(n_experts + 1) * sizeof(int), stream>>>(counts, n_experts, tile_rows, first,
                                                                              tile_map, n_tiles);
    int rc = mx_launch_status();
    if (rc != MX_OK) return rc;
    moe_scatter_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(ids, place, first, order, n_pairs, n_experts);
    return mx_launch_status();
}

// glu != 0: a = the tokens' activations [tokens][lda], source row of sorted row r is order[r] / a_div, w holds per
// expert 2 N rows (gate, then up), out [pairs][N] in the operand type by sorted row. glu == 0: a = [pairs][lda] by
// sorted row, out float [pairs][N] by pair, times pair_weight. `max_tiles` bounds the tiles a step can have.
extern "C" int mx_moe_gemm(const void* a, int dtype, int lda, const int* order, int a_div, const void* w,
                           long long expert_stride, int N, int K, const int* tile_map, const int* n_tiles, int max_tiles,
                           void* out, const float* pair_weight, int glu, int act, float limit, float slope, float shift,
                           cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return MX_OK;
    if (max_tiles > 65535) MX_REFUSE("routed feed-forward: %d row tiles exceed the grid", max_tiles);
    const dim3 grid((N + MOE_BN - 1) / MOE_BN, max_tiles);
    const ClampedAct clamped{limit, slope, shift};
    if (glu && (act < 0 || act > 2)) MX_REFUSE("routed feed-forward: activation %d", act);
#define MOE_LAUNCH(T, GLU, ACT)                                                                                        \
    moe_gemm_kernel<T, GLU, ACT><<<grid, 256, 0, stream>>>((const T*)a, lda, order, a_div, (const T*)w, expert_stride, \
                                                           N, K, tile_map, n_tiles, out, pair_weight, clamped)
    if (dtype == MX_DTYPE_F32) {
        if (!glu) MOE_LAUNCH(float, false, 0);
        else if (act == 0) MOE_LAUNCH(float, true, 0);
        else if (act == 1) MOE_LAUNCH(float, true, 1);
        else MOE_LAUNCH(float, true, 2);
    } else {
        if (!glu) MOE_LAUNCH(__nv_bfloat16, false, 0);
        else if (act == 0) MOE_LAUNCH(__nv_bfloat16, true, 0);
        else if (act == 1) MOE_LAUNCH(__nv_bfloat16, true, 1);
        else MOE_LAUNCH(__nv_bfloat16, true, 2);
    }
#undef MOE_LAUNCH
    return mx_launch_status();
}

extern "C" int mx_moe_gather(const void* h, int ld, const int* order, int top, void* sorted, int n_pairs, int K,
                             cudaStream_t stream) {
    if (n_pairs <= 0) return MX_OK;
    if (K % 8 != 0 || ld % 8 != 0 || ((uintptr_t)h | (uintptr_t)sorted) % 16 != 0)
        MX_REFUSE("routed feed-forward: gathered rows must be 16-byte aligned (K = %d, stride %d)", K, ld);
    const long long count = (long long)n_pairs * (K / 8);
    moe_gather_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)h, ld, order, top, (__nv_bfloat16*)sorted, K / 8, count);
    return mx_launch_status();
}

extern "C" int mx_moe_combine_sorted(const float* rows, const int* ids, const int* place, const int* first,
                                     const float* weight, float* residual, int n_tokens, int top, int width,
                                     const void* input, int input_dtype, int input_ld, int n_experts,
                                     cudaStream_t stream) {
    const long long count = (long long)n_tokens * width;
    if (count <= 0) return MX_OK;
    if (input == nullptr) n_experts = 0x7fffffff;          // every pair has a row
    const bool f32 = input == nullptr || input_dtype == MX_DTYPE_F32;
    if (width % 4 == 0 && ((uintptr_t)rows | (uintptr_t)residual | (uintptr_t)input) % 16 == 0 && input_ld % 4 == 0) {
        const long long count4 = count / 4;
        const unsigned blocks = (unsigned)((count4 + 255) / 256);
        if (f32)
            moe_combine_sorted_vec_kernel<float><<<blocks, 256, 0, stream>>>(
                rows, ids, place, first, weight, residual, top, width / 4, count4, (const float*)input, input_ld, n_experts);
        else
            moe_combine_sorted_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
                rows, ids, place, first, weight, residual, top, width / 4, count4, (const __nv_bfloat16*)input, input_ld,
                n_experts);
        return mx_launch_status();
    }
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (f32)
        moe_combine_sorted_kernel<float><<<blocks, 256, 0, stream>>>(
            rows, ids, place, first, weight, residual, top, width, count, (const float*)input, input_ld, n_experts);
    else
        moe_combine_sorted_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            rows, ids, place, first, weight, residual, top, width, count, (const __nv_bfloat16*)input, input_ld, n_experts);
    return mx_launch_status();
}

extern "C" int mx_moe_combine(const float* pairs, float* residual, int n_tokens, int top, int width, const int* ids,
                              const float* weight, const void* input, int input_dtype, int input_ld, int n_experts,
                              cudaStream_t stream) {
    const long long count = (long long)n_tokens * width;
    if (count <= 0) return MX_OK;
    if (input == nullptr || weight == nullptr) ids = nullptr;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (input == nullptr || input_dtype == MX_DTYPE_F32)
        moe_combine_kernel<float><<<blocks, 256, 0, stream>>>(pairs, residual, top, width, count, ids, weight,
                                                              (const float*)input, input_ld, n_experts);
    else
        moe_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(pairs, residual, top, width, count, ids, weight,
                                                                      (const __nv_bfloat16*)input, input_ld, n_experts);
    return mx_launch_status();
}

// out = act(gate) * up on rows [gate (ff) | up (ff)]; act 0 = gelu (tanh form), 1 = silu
extern "C" int mx_glu(const void* gu, int ld, void* out, int dtype, int n_tokens, int ff, int act, cudaStream_t stream) {
    const long long count = (long long)n_tokens * ff;
    if (count <= 0) return MX_OK;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == MX_DTYPE_BF16 && ff % 8 == 0 && ld % 8 == 0 && ((uintptr_t)gu | (uintptr_t)out) % 16 == 0) {
        const long long groups = count >> 3;
        glu_vec_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, ld,
                                                                             (__nv_bfloat16*)out, ff, act, groups);
        return mx_launch_status();
    }
    if (dtype == MX_DTYPE_F32)
        glu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, ld, (float*)out, ff, act, count);
    else
        glu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, ld, (__nv_bfloat16*)out, ff, act,
                                                             count);
    return mx_launch_status();
}
