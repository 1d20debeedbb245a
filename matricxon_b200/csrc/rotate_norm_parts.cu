// The step ahead of an attention whose queries and keys are rotated over a part of the head and then divided by
// their root mean square, head by head, without a learned weight.
//
// mx_rotate_norm_kv_write: the float result of a fused projection, rows
//   [q heads x dim | k heads x dim | v heads x vdim | ...], becomes the operands of the paged attention kernels:
//     q_out [tokens][heads * hd]                 q_h rotated over its first `rot` entries, then q_h / rms(q_h); tail zero
//     cache keys   [page][0][kv head][slot][hd]  k_h the same way, tail zero
//     cache values [page][1][kv head][hd][slot]  v_h as it is, tail (vdim..hd) zero
//   Rotation pairs entry i with entry i + rot/2 (i < rot/2): (u, v) -> (u cos a - v sin a, v cos a + u sin a),
//   a = position * freq[i] in float. rms(x) = sqrt(mean over the head's `dim` entries of x^2 + eps), taken of the
//   rotated head in float; eps < 0 leaves the heads as they are. A warp owns a head (up to 256 entries in
//   registers); blockIdx.y shares a token's heads out between blocks when tokens are few.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int RN_THREADS = 128, RN_WARPS = RN_THREADS / 32, RN_SLOTS = 8;      // heads of up to 32 * RN_SLOTS entries

template <typename T>
__global__ void __launch_bounds__(RN_THREADS)
rotate_norm_kv_write_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ positions,
                            const float* __restrict__ freq, int rot, float eps, const int* __restrict__ slots,
                            T* __restrict__ cache, long long n_slots, int page_size, T* __restrict__ q_out, int n_heads,
                            int n_kv_heads, int dim, int vdim, int hd, int* status) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int half = rot >> 1;
    long long slot = slots ? slots[t] : -1;
    if (slot != -1 && (slot < 0 || slot >= n_slots)) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const size_t head_stride = (size_t)page_size * hd;
    T* kbase = cache + ((size_t)page * 2 * n_kv_heads) * head_stride + (size_t)offset * hd;
    T* vbase = cache + ((size_t)page * 2 * n_kv_heads + n_kv_heads) * head_stride + offset;
    const int heads = n_heads + (slot >= 0 ? n_kv_heads : 0);
    for (int h = blockIdx.y * RN_WARPS + warp; h < heads; h += gridDim.y * RN_WARPS) {
        const float* src = row + (size_t)h * dim;            // k heads follow the q heads directly
        float value[RN_SLOTS];
        float squares = 0.f;
#pragma unroll
        for (int j = 0; j < RN_SLOTS; ++j) {
            const int d = lane + 32 * j;
            float v = 0.f;
            if (d < rot) {
                const int i = d < half ? d : d - half;
                float s, c;
                sincosf(pos * freq[i], &s, &c);
                v = d < half ? src[d] * c - src[d + half] * s : src[d] * c + src[d - half] * s;
            } else if (d < dim) {
                v = src[d];
            }
            value[j] = v;
            squares = fmaf(v, v, squares);
        }
        const float inv = eps >= 0.f ? 1.0f / sqrtf(warp_sum(squares) / (float)dim + eps) : 1.f;
        T* dst = h < n_heads ? q_out + ((size_t)t * n_heads + h) * hd : kbase + (size_t)(h - n_heads) * head_stride;
#pragma unroll
        for (int j = 0; j < RN_SLOTS; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) dst[d] = from_float<T>(value[j] * inv);
        }
    }
    if (slot < 0) return;
    const float* vrow = row + (size_t)(n_heads + n_kv_heads) * dim;
    for (int item = blockIdx.y * RN_THREADS + threadIdx.x; item < n_kv_heads * hd; item += gridDim.y * RN_THREADS) {
        const int h = item / hd, d = item - h * hd;
        const float value = d < vdim ? vrow[(size_t)h * vdim + d] : 0.f;
        vbase[(size_t)h * head_stride + (size_t)d * page_size] = from_float<T>(value);
    }
}

}  // namespace

extern "C" int mx_rotate_norm_kv_write(const float* proj, int ld, const int* positions, const float* freq, int rot,
                                       float eps, const int* slots, void* cache, long long n_pages, int page_size,
                                       void* q_out, int dtype, int n_tokens, int n_heads, int n_kv_heads, int dim,
                                       int vdim, int hd, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (hd < dim || hd < vdim) MX_REFUSE("attention operands: a padded head of %d holds neither %d nor %d", hd, dim, vdim);
    if (hd > 32 * RN_SLOTS) MX_REFUSE("attention operands: a head of %d entries (at most %d)", hd, 32 * RN_SLOTS);
    if (rot < 0 || rot % 2 != 0 || rot > dim) MX_REFUSE("attention operands: %d rotated entries in a head of %d", rot, dim);
    if (ld < (n_heads + n_kv_heads) * dim + n_kv_heads * vdim) MX_REFUSE("attention operands: projection rows are too short");
    const long long n_slots = n_pages * page_size;
    const int pieces = n_tokens >= 512 ? 1 : max(1, min(32, (n_heads + n_kv_heads + RN_WARPS - 1) / RN_WARPS));
    const dim3 grid(n_tokens, pieces);
    if (dtype == MX_DTYPE_F32)
        rotate_norm_kv_write_kernel<float><<<grid, RN_THREADS, 0, stream>>>(
            proj, ld, positions, freq, rot, eps, cache ? slots : nullptr, (float*)cache, n_slots, page_size, (float*)q_out,
            n_heads, n_kv_heads, dim, vdim, hd, status);
    else
        rotate_norm_kv_write_kernel<__nv_bfloat16><<<grid, RN_THREADS, 0, stream>>>(
            proj, ld, positions, freq, rot, eps, cache ? slots : nullptr, (__nv_bfloat16*)cache, n_slots, page_size,
            (__nv_bfloat16*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    return mx_launch_status();
}
