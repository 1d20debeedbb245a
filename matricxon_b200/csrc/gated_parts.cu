// Small fused steps around attention and feed-forward products.
//
// mx_qk_norm_kv_write: the float result of a fused projection, rows [q heads x dim | k heads x dim |
//   v heads x vdim | ...], becomes the operands of the paged attention kernels:
//     q_out [tokens][heads * hd]   unit(q_h) * q_weight per head (hd >= dim, vdim; the tail is zero)
//     cache keys   [page][0][kv head][slot][hd]   unit(k_h) * k_weight, tail zero
//     cache values [page][1][kv head][hd][slot]   v_h, tail zero
//   unit(x) = x / sqrt(mean(x^2) + eps) over the head's `dim` elements, in float; with null
//   weights the heads pass unnormalised. No rotation: positions do not enter. One block per token,
//   one warp per head at a time.
// mx_sigmoid_gate: out[t][h * vdim + e] = attn[t][h * hd + e] * sigmoid(gate[t][h * vdim + e]),
//   gate in float (a column range of the same fused projection), the product rounded once.
// mx_clamped_glu: the activation of a gated feed-forward whose fused first product gives rows
//   [gate (ff) | up (ff)]: g = min(gate, limit), u = clamp(up, -limit, limit),
//   out = g * sigmoid(slope * g) * (u + shift); limit <= 0 switches the clamps off.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_kv_write_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ q_weight,
                        const float* __restrict__ k_weight, float eps, const int* __restrict__ slots,
                        T* __restrict__ cache, long long n_slots, int page_size, T* __restrict__ q_out,
                        int n_heads, int n_kv_heads, int dim, int vdim, int hd, int* status) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float* row = proj + (size_t)t * ld;
    long long slot = slots ? slots[t] : -1;
    if (slot != -1 && (slot < 0 || slot >= n_slots)) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const size_t head_stride = (size_t)page_size * hd;
    T* kbase = cache + ((size_t)page * 2 * n_kv_heads) * head_stride + (size_t)offset * hd;
    T* vbase = cache + ((size_t)page * 2 * n_kv_heads + n_kv_heads) * head_stride + offset;
    const int norm_heads = n_heads + (slot >= 0 ? n_kv_heads : 0);
    for (int h = warp; h < norm_heads; h += n_warps) {
        const bool is_q = h < n_heads;
        const float* src = row + (size_t)h * dim;            // k heads follow the q heads directly
        const float* w = is_q ? q_weight : k_weight;
        float inv = 1.f;
        if (w) {
            float s = 0.f;
            for (int d = lane; d < dim; d += 32) s = fmaf(src[d], src[d], s);
            inv = 1.0f / sqrtf(warp_sum(s) / (float)dim + eps);
        }
        T* dst = is_q ? q_out + ((size_t)t * n_heads + h) * hd : kbase + (size_t)(h - n_heads) * head_stride;
        for (int d = lane; d < hd; d += 32)
            dst[d] = from_float<T>(d < dim ? (w ? src[d] * inv * w[d] : src[d]) : 0.f);
    }
    if (slot < 0) return;
    const float* vrow = row + (size_t)(n_heads + n_kv_heads) * dim;
    for (int item = threadIdx.x; item < n_kv_heads * hd; item += blockDim.x) {
        const int h = item / hd, d = item - h * hd;
        vbase[(size_t)h * head_stride + (size_t)d * page_size] =
            from_float<T>(d < vdim ? vrow[(size_t)h * vdim + d] : 0.f);
    }
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ attn, const float* __restrict__ gate, int gate_ld,
                                    T* __restrict__ out, int n_heads, int vdim, int hd, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int width = n_heads * vdim;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const int h = c / vdim, e = c - h * vdim;
    const float a = to_float(attn[((size_t)t * n_heads + h) * hd + e]);
    out[i] = from_float<T>(a * sigmoidf_(gate[(size_t)t * gate_ld + c]));
}

// eight neighbouring columns a thread for bfloat16 rows whose widths are multiples of 8: one 16-byte load of the
// heads' values, two of the float gates, one 16-byte store
__global__ void sigmoid_gate_vec_kernel(const __nv_bfloat16* __restrict__ attn, const float* __restrict__ gate,
                                        int gate_ld, __nv_bfloat16* __restrict__ out, int n_heads, int vdim, int hd,
                                        long long count8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count8) return;
    const int width8 = n_heads * vdim / 8;
    const long long t = i / width8;
    const int c = (int)(i - t * width8) * 8;
    const int h = c / vdim, e = c - h * vdim;
    const uint4 raw = *reinterpret_cast<const uint4*>(attn + ((size_t)t * n_heads + h) * hd + e);
    const float4 g0 = *reinterpret_cast<const float4*>(gate + (size_t)t * gate_ld + c);
    const float4 g1 = *reinterpret_cast<const float4*>(gate + (size_t)t * gate_ld + c + 4);
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint4 packed;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 v = __bfloat1622float2(a[k]);
        o[k] = __floats2bfloat162_rn(v.x * sigmoidf_(g[2 * k]), v.y * sigmoidf_(g[2 * k + 1]));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * n_heads * vdim + c) = packed;
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int ff,
                                   float limit, float slope, float shift, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const long long t = i / ff;
    const int c = (int)(i - t * ff);
    float g = to_float(gu[(size_t)t * ld + c]);
    float u = to_float(gu[(size_t)t * ld + ff + c]);
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    out[i] = from_float<T>(g * sigmoidf_(slope * g) * (u + shift));
}

// eight neighbouring columns a thread, 16-byte accesses (bfloat16 rows whose width and stride are multiples of 8)
__global__ void clamped_glu_vec_kernel(const __nv_bfloat16* __restrict__ gu, int ld, __nv_bfloat16* __restrict__ out,
                                       int ff, float limit, float slope, float shift, long long groups) {
    pdl_trigger();
    pdl_wait();
    gu = after_wait(gu);
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
        float g[2] = {__low2float(g2[e]), __high2float(g2[e])};
        float u[2] = {__low2float(u2[e]), __high2float(u2[e])};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (limit > 0.f) {
                g[k] = fminf(g[k], limit);
                u[k] = fminf(fmaxf(u[k], -limit), limit);
            }
            g[k] = g[k] * sigmoidf_(slope * g[k]) * (u[k] + shift);
        }
        o2[e] = __floats2bfloat162_rn(g[0], g[1]);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ff + c) = oraw;
}

}  // namespace

extern "C" int mx_qk_norm_kv_write(const float* proj, int ld, const float* q_weight, const float* k_weight,
                                   float eps, const int* slots, void* cache, long long n_pages, int page_size,
                                   void* q_out, int dtype, int n_tokens, int n_heads, int n_kv_heads, int dim,
                                   int vdim, int hd, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (hd < dim || hd < vdim) MX_REFUSE("attention operands: a padded head of %d holds neither %d nor %d", hd, dim, vdim);
    if (ld < (n_heads + n_kv_heads) * dim + n_kv_heads * vdim) MX_REFUSE("attention operands: projection rows are too short");
    const long long n_slots = n_pages * page_size;
    if (dtype == MX_DTYPE_F32)
        qk_norm_kv_write_kernel<float><<<n_tokens, 128, 0, stream>>>(
            proj, ld, q_weight, k_weight, eps, cache ? slots : nullptr, (float*)cache, n_slots, page_size,
            (float*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    else
        qk_norm_kv_write_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>(
            proj, ld, q_weight, k_weight, eps, cache ? slots : nullptr, (__nv_bfloat16*)cache, n_slots, page_size,
            (__nv_bfloat16*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    return mx_launch_status();
}

extern "C" int mx_sigmoid_gate(const void* attn, const float* gate, int gate_ld, void* out, int dtype,
                               int n_tokens, int n_heads, int vdim, int hd, cudaStream_t stream) {
    const long long count = (long long)n_tokens * n_heads * vdim;
    if (count <= 0) return MX_OK;
    if (dtype == MX_DTYPE_BF16 && vdim % 8 == 0 && hd % 8 == 0 && gate_ld % 4 == 0 && ((uintptr_t)attn % 16 == 0) &&
        ((uintptr_t)out % 16 == 0) && ((uintptr_t)gate % 16 == 0)) {
        const long long count8 = count / 8;
        sigmoid_gate_vec_kernel<<<(unsigned)((count8 + 255) / 256), 256, 0, stream>>>(
            (const __nv_bfloat16*)attn, gate, gate_ld, (__nv_bfloat16*)out, n_heads, vdim, hd, count8);
        return mx_launch_status();
    }
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == MX_DTYPE_F32)
        sigmoid_gate_kernel<float><<<blocks, 256, 0, stream>>>((const float*)attn, gate, gate_ld, (float*)out,
                                                              n_heads, vdim, hd, count);
    else
        sigmoid_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)attn, gate, gate_ld, (__nv_bfloat16*)out, n_heads, vdim, hd, count);
    return mx_launch_status();
}

extern "C" int mx_clamped_glu(const void* gu, int ld, void* out, int dtype, int n_tokens, int ff, float limit,
                              float slope, float shift, cudaStream_t stream) {
    const long long count = (long long)n_tokens * ff;
    if (count <= 0) return MX_OK;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == MX_DTYPE_BF16 && ff % 8 == 0 && ld % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        const long long groups = count >> 3;
        mx_launch_chained(clamped_glu_vec_kernel, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, stream,
                          (const __nv_bfloat16*)gu, ld, (__nv_bfloat16*)out, ff, limit, slope, shift, groups);
        return mx_launch_status();
    }
    if (dtype == MX_DTYPE_F32)
        clamped_glu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, ld, (float*)out, ff, limit, slope,
                                                             shift, count);
    else
        clamped_glu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, ld,
                                                                     (__nv_bfloat16*)out, ff, limit, slope, shift,
                                                                     count);
    return mx_launch_status();
}
