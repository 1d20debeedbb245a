// The end of a sublayer whose own output is normalised before it joins the residual stream, and a small
// input that a layer takes from the token itself.
//
// mx_layernorm_scaled_add: x[r] += LayerNorm(y[r]) * weight (+ bias) then * scale, entry by entry, where
//   LayerNorm(y) = (y - mean) / sqrt(mean of squared deviations + eps); statistics in float with two passes over the
//   row held in registers (rows that are no multiple of 4 or too long: in shared memory). `scale` (a vector, may be
//   null) is the layer's learned scale of the branch. `act` (may be null) receives the new x in bfloat16 or float:
//   the next sublayer's input, so that no rounding pass follows.
//   `centre` 0 leaves the mean in: x[r] += y / sqrt(mean(y^2) + eps) * weight, the root-mean-square form.
// mx_gelu_gate_rows: g[t][d] = gelu_tanh(z[t][d]) * table[token id][col0 + d], the middle of the token input when its
//   two products run as matrix products (wide layers); mx_token_side_input is the whole of it in one kernel.
// mx_scale_rows: x *= s (the constant some models put on their logits).
// mx_token_side_input: per token t and layer, with e = table[token id][col0 .. col0 + dim):
//     g = gelu_tanh(G x_t) * e            G [dim][hidden]
//     y = P g                             P [hidden][dim]
//     x_t += y / sqrt(mean(y^2) + eps) * norm
//   all in float (weights in T); `act` as above. TS_TOKENS tokens share a block, so that G and P are read once for
//   all of them: a warp per row of G forms the tokens' dot products together, a thread per column of x the tokens'
//   y entries together.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int BN_VPT = 8;          // float4 vectors a thread holds at most

template <typename TAct, int THREADS>
__global__ void __launch_bounds__(THREADS)
layernorm_scaled_add_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ weight,
                                const float* __restrict__ bias, const float* __restrict__ scale, TAct* __restrict__ act,
                                int hidden, float eps, int centre) {
    __shared__ float scratch[32];
    const int r = blockIdx.x, n_vec = hidden >> 2;
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * hidden);
    float4 v[BN_VPT];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < BN_VPT; ++j) {
        const int i = threadIdx.x + j * THREADS;
        v[j] = i < n_vec ? yr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = centre ? block_sum(s, scratch) / (float)hidden : 0.f;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < BN_VPT; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i < n_vec) {
            v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
            q += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
        }
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * hidden);
#pragma unroll
    for (int j = 0; j < BN_VPT; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i >= n_vec) continue;
        const float4 w = reinterpret_cast<const float4*>(weight)[i];
        float4 o = make_float4(v[j].x * rstd * w.x, v[j].y * rstd * w.y, v[j].z * rstd * w.z, v[j].w * rstd * w.w);
        if (bias) {
            const float4 b = reinterpret_cast<const float4*>(bias)[i];
            o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
        }
        if (scale) {
            const float4 c = reinterpret_cast<const float4*>(scale)[i];
            o.x *= c.x; o.y *= c.y; o.z *= c.z; o.w *= c.w;
        }
        float4 xv = xr[i];
        xv.x += o.x; xv.y += o.y; xv.z += o.z; xv.w += o.w;
        xr[i] = xv;
        if (act) {
            TAct* a = act + (size_t)r * hidden + 4 * (size_t)i;
            a[0] = from_float<TAct>(xv.x); a[1] = from_float<TAct>(xv.y);
            a[2] = from_float<TAct>(xv.z); a[3] = from_float<TAct>(xv.w);
        }
    }
}

template <typename TAct>
__global__ void layernorm_scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y,
                                            const float* __restrict__ weight, const float* __restrict__ bias,
                                            const float* __restrict__ scale, TAct* __restrict__ act, int hidden,
                                            float eps, int centre) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* yr = y + (size_t)r * hidden;
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = yr[i];
        row_cache[i] = v;
        s += v;
    }
    const float mean = centre ? block_sum(s, scratch) / (float)hidden : 0.f;
    float q = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_cache[i] - mean;
        q += d * d;
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float o = (row_cache[i] - mean) * rstd * weight[i];
        if (bias) o += bias[i];
        if (scale) o *= scale[i];
        const float xv = x[(size_t)r * hidden + i] + o;
        x[(size_t)r * hidden + i] = xv;
        if (act) act[(size_t)r * hidden + i] = from_float<TAct>(xv);
    }
}

__global__ void scale_rows_kernel(float* __restrict__ x, long long count, float s) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] *= s;
}

// out[t][d] = gelu_tanh(z[t][d]) * table[id_t][col0 + d]: what the token brings, gated by the stream's projection
template <typename T>
__global__ void gelu_gate_rows_kernel(const float* __restrict__ z, int ld, const int* __restrict__ token_ids,
                                      const T* __restrict__ table, int table_ld, int col0, int vocab, T* __restrict__ out,
                                      int n_tokens, int dim, int* status) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * dim) return;
    const int t = (int)(i / dim), d = (int)(i - (long long)t * dim);
    const int id = token_ids[t];
    float e = 0.f;
    if (id >= 0 && id < vocab) e = to_float(table[(size_t)id * table_ld + col0 + d]);
    else if (d == 0) atomicOr(status, MX_STATUS_BAD_TOKEN_ID);
    out[i] = from_float<T>(gelu_tanh(z[(size_t)t * ld + d]) * e);
}

constexpr int TS_TOKENS = 4;       // tokens a block handles together
constexpr int TS_COLS = 8;         // columns of x a thread owns at most

template <typename T, typename TAct>
__global__ void __launch_bounds__(1024)
token_side_input_kernel(float* __restrict__ x, TAct* __restrict__ act, const int* __restrict__ token_ids,
                        const T* __restrict__ table, int table_ld, int col0, int vocab, const T* __restrict__ gate,
                        const T* __restrict__ proj, const float* __restrict__ norm, int n_tokens, int hidden, int dim,
                        float eps, int* status) {
    extern __shared__ __align__(16) float side_s[];
    float* x_s = side_s;                                   // [TS_TOKENS][hidden]
    float* g_s = x_s + TS_TOKENS * hidden;                 // [TS_TOKENS][dim]
    __shared__ float scratch[32];
    const int t0 = blockIdx.x * TS_TOKENS, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_here = min(TS_TOKENS, n_tokens - t0);
    for (int i = tid; i < TS_TOKENS * hidden; i += blockDim.x) {
        const int k = i / hidden;
        x_s[i] = k < n_here ? x[(size_t)(t0 + k) * hidden + (i - k * hidden)] : 0.f;
    }
    __syncthreads();
    // g = gelu_tanh(G x) * e: a warp per row of G, the tokens' sums side by side
    for (int d = warp; d < dim; d += blockDim.x >> 5) {
        const T* grow = gate + (size_t)d * hidden;
        float z[TS_TOKENS] = {};
        for (int c = lane; c < hidden; c += 32) {
            const float w = to_float(grow[c]);
#pragma unroll
            for (int k = 0; k < TS_TOKENS; ++k) z[k] = fmaf(w, x_s[k * hidden + c], z[k]);
        }
#pragma unroll
        for (int k = 0; k < TS_TOKENS; ++k) {
            const float total = warp_sum(z[k]);
            if (lane == 0 && k < n_here) {
                const int id = token_ids[t0 + k];
                float e = 0.f;
                if (id >= 0 && id < vocab) e = to_float(table[(size_t)id * table_ld + col0 + d]);
                else atomicOr(status, MX_STATUS_BAD_TOKEN_ID);
                g_s[k * dim + d] = gelu_tanh(total) * e;
            }
        }
    }
    __syncthreads();
    // y = P g: a thread per column, the tokens' entries side by side
    float yv[TS_COLS][TS_TOKENS];
    float squares[TS_TOKENS] = {};
#pragma unroll
    for (int j = 0; j < TS_COLS; ++j) {
        const int c = tid + j * blockDim.x;
#pragma unroll
        for (int k = 0; k < TS_TOKENS; ++k) yv[j][k] = 0.f;
        if (c < hidden) {
            const T* prow = proj + (size_t)c * dim;
            for (int d = 0; d < dim; ++d) {
                const float w = to_float(prow[d]);
#pragma unroll
                for (int k = 0; k < TS_TOKENS; ++k) yv[j][k] = fmaf(w, g_s[k * dim + d], yv[j][k]);
            }
#pragma unroll
            for (int k = 0; k < TS_TOKENS; ++k) squares[k] = fmaf(yv[j][k], yv[j][k], squares[k]);
        }
    }
    float inv[TS_TOKENS];
#pragma unroll
    for (int k = 0; k < TS_TOKENS; ++k) inv[k] = 1.0f / sqrtf(block_sum(squares[k], scratch) / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < TS_COLS; ++j) {
        const int c = tid + j * blockDim.x;
        if (c >= hidden) continue;
        const float w = norm[c];
#pragma unroll
        for (int k = 0; k < TS_TOKENS; ++k) {
            if (k >= n_here) continue;
            const float xv = x_s[k * hidden + c] + yv[j][k] * inv[k] * w;
            x[(size_t)(t0 + k) * hidden + c] = xv;
            if (act) act[(size_t)(t0 + k) * hidden + c] = from_float<TAct>(xv);
        }
    }
}

}  // namespace

extern "C" int mx_layernorm_scaled_add(float* x, const float* y, const float* weight, const float* bias,
                                       const float* scale, void* act, int act_dtype, int n_rows, int hidden, float eps,
                                       int centre, cudaStream_t stream) {
    if (n_rows <= 0 || hidden <= 0) return MX_OK;
    const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)scale) & 15) == 0;
    const bool f32 = act_dtype == MX_DTYPE_F32;
    if (hidden % 4 == 0 && aligned && hidden <= 4 * BN_VPT * 512) {
        const int n_vec = hidden / 4;
        if (n_vec <= BN_VPT * 128) {
            if (f32) layernorm_scaled_add_vec_kernel<float, 128><<<n_rows, 128, 0, stream>>>(x, y, weight, bias, scale, (float*)act, hidden, eps, centre);
            else layernorm_scaled_add_vec_kernel<__nv_bfloat16, 128><<<n_rows, 128, 0, stream>>>(x, y, weight, bias, scale, (__nv_bfloat16*)act, hidden, eps, centre);
        } else {
            if (f32) layernorm_scaled_add_vec_kernel<float, 512><<<n_rows, 512, 0, stream>>>(x, y, weight, bias, scale, (float*)act, hidden, eps, centre);
            else layernorm_scaled_add_vec_kernel<__nv_bfloat16, 512><<<n_rows, 512, 0, stream>>>(x, y, weight, bias, scale, (__nv_bfloat16*)act, hidden, eps, centre);
        }
        return mx_launch_status();
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) MX_REFUSE("norm of a branch: rows of %d entries", hidden);
    if (f32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_scaled_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_scaled_add_kernel<float><<<n_rows, 256, smem, stream>>>(x, y, weight, bias, scale, (float*)act, hidden, eps, centre);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_scaled_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        layernorm_scaled_add_kernel<__nv_bfloat16><<<n_rows, 256, smem, stream>>>(x, y, weight, bias, scale, (__nv_bfloat16*)act, hidden, eps, centre);
    }
    return mx_launch_status();
}

extern "C" int mx_scale_rows(float* x, long long count, float s, cudaStream_t stream) {
    if (count <= 0) return MX_OK;
    scale_rows_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(x, count, s);
    return mx_launch_status();
}

template <typename T, typename TAct>
static int launch_token_side(float* x, void* act, const int* token_ids, const void* table, int table_ld, int col0,
                             int vocab, const void* gate, const void* proj, const float* norm, int n_tokens, int hidden,
                             int dim, float eps, int* status, cudaStream_t stream) {
    const int threads = hidden <= 256 ? 128 : (hidden <= 2048 ? 256 : 1024);
    if (hidden > threads * TS_COLS) MX_REFUSE("token input: rows of %d entries", hidden);
    const size_t smem = (size_t)TS_TOKENS * (hidden + dim) * sizeof(float);
    if (smem > 200 * 1024) MX_REFUSE("token input: %zu bytes of shared memory", smem);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(token_side_input_kernel<T, TAct>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    token_side_input_kernel<T, TAct><<<(n_tokens + TS_TOKENS - 1) / TS_TOKENS, threads, smem, stream>>>(
        x, (TAct*)act, token_ids, (const T*)table, table_ld, col0, vocab, (const T*)gate, (const T*)proj, norm, n_tokens,
        hidden, dim, eps, status);
    return mx_launch_status();
}

// `dtype` is the type of table and out.
extern "C" int mx_gelu_gate_rows(const float* z, int ld, const int* token_ids, const void* table, int table_ld, int col0,
                                 int vocab, void* out, int dtype, int n_tokens, int dim, int* status,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (dim <= 0 || col0 < 0 || col0 + dim > table_ld || ld < dim) MX_REFUSE("token input: columns %d..%d of a table of %d", col0, col0 + dim, table_ld);
    const long long count = (long long)n_tokens * dim;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == MX_DTYPE_F32)
        gelu_gate_rows_kernel<float><<<blocks, 256, 0, stream>>>(z, ld, token_ids, (const float*)table, table_ld, col0, vocab,
                                                                 (float*)out, n_tokens, dim, status);
    else
        gelu_gate_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(z, ld, token_ids, (const __nv_bfloat16*)table,
                                                                         table_ld, col0, vocab, (__nv_bfloat16*)out,
                                                                         n_tokens, dim, status);
    return mx_launch_status();
}

// `dtype` is the type of table, gate and proj; `act` (may be null) has the same type.
extern "C" int mx_token_side_input(float* x, void* act, const int* token_ids, const void* table, int table_ld, int col0,
                                   int vocab, const void* gate, const void* proj, const float* norm, int dtype,
                                   int n_tokens, int hidden, int dim, float eps, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (dim <= 0 || col0 < 0 || col0 + dim > table_ld) MX_REFUSE("token input: columns %d..%d of a table of %d", col0, col0 + dim, table_ld);
    if (dtype == MX_DTYPE_F32)
        return launch_token_side<float, float>(x, act, token_ids, table, table_ld, col0, vocab, gate, proj, norm, n_tokens,
                                               hidden, dim, eps, status, stream);
    return launch_token_side<__nv_bfloat16, __nv_bfloat16>(x, act, token_ids, table, table_ld, col0, vocab, gate, proj, norm,
                                                           n_tokens, hidden, dim, eps, status, stream);
}
