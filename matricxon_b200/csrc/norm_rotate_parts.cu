// The step ahead of an attention whose queries and keys are RMS-normalised head by head with a learned weight and
// then rotated over a part of the head.
//
// mx_norm_rotate_kv_write: the float result of a fused projection, rows
//   [q heads x dim | k heads x dim | v heads x vdim | ...], becomes the operands of the paged attention kernels:
//     q_out [tokens][heads * hd]                 n(q_h) rotated over its first `rot` entries; tail (dim..hd) zero
//     cache keys   [page][0][kv head][slot][hd]  n(k_h) the same way, tail zero
//     cache values [page][1][kv head][hd][slot]  v_h as it is, tail (vdim..hd) zero
//   n(x) = x / sqrt(mean over the head's `dim` entries of x^2 + eps) * w, with one weight vector for all query heads
//   and one for all key heads (null: the head is left as it is). The rotation comes after the norm and pairs entry
//   i with entry i + rot/2 or, `interleaved`, entry 2i with entry 2i + 1 (i < rot/2):
//   (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq[i] in float; a token's cosines and sines
//   are formed once per block, in shared memory.
//   A warp owns a head (up to 256 entries in registers); blockIdx.y shares a token's heads out between blocks when
//   tokens are few.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int NR_THREADS = 128, NR_WARPS = NR_THREADS / 32, NR_SLOTS = 8;      // heads of up to 32 * NR_SLOTS entries

template <typename T>
__global__ void __launch_bounds__(NR_THREADS)
norm_rotate_kv_write_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ positions,
                            const float* __restrict__ freq, int rot, int interleaved,
                            const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                            const int* __restrict__ slots, T* __restrict__ cache, long long n_slots, int page_size,
                            T* __restrict__ q_out, int n_heads, int n_kv_heads, int dim, int vdim, int hd, int* status) {
    extern __shared__ float cs[];                           // cos[half], sin[half] of the token's angles
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float pos = (float)positions[t];                  // step metadata and constants: no kernel writes them
    const int half = rot >> 1;
    // every head of the token turns by the same angles: once per block, not once per entry
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freq[i], &cs[half + i], &cs[i]);
    __syncthreads();
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
    pdl_wait();
    const float* row = after_wait(proj) + (size_t)t * ld;
    for (int h = blockIdx.y * NR_WARPS + warp; h < heads; h += gridDim.y * NR_WARPS) {
        const float* src = row + (size_t)h * dim;            // k heads follow the q heads directly
        const float* weight = h < n_heads ? q_weight : k_weight;
        float raw[NR_SLOTS];
        float squares = 0.f;
#pragma unroll
        for (int j = 0; j < NR_SLOTS; ++j) {
            const int d = lane + 32 * j;
            raw[j] = d < dim ? src[d] : 0.f;
            squares = fmaf(raw[j], raw[j], squares);
        }
        const float inv = weight ? 1.0f / sqrtf(warp_sum(squares) / (float)dim + eps) : 1.f;
        T* dst = h < n_heads ? q_out + ((size_t)t * n_heads + h) * hd : kbase + (size_t)(h - n_heads) * head_stride;
#pragma unroll
        for (int j = 0; j < NR_SLOTS; ++j) {
            const int d = lane + 32 * j;
            if (d >= hd) continue;
            float v = weight && d < dim ? raw[j] * inv * weight[d] : raw[j];
            if (d < rot) {
                // the partner's normalised value is formed from the projection again: it lives in another lane or slot
                const int i = interleaved ? d >> 1 : (d < half ? d : d - half);
                const bool first = interleaved ? !(d & 1) : d < half;
                const int other = interleaved ? d ^ 1 : (first ? d + half : d - half);
                const float u = weight ? src[other] * inv * weight[other] : src[other];
                const float c = cs[i], s = cs[half + i];
                v = first ? v * c - u * s : v * c + u * s;
            }
            dst[d] = from_float<T>(v);
        }
    }
    if (slot < 0) return;
    const float* vrow = row + (size_t)(n_heads + n_kv_heads) * dim;
    for (int item = blockIdx.y * NR_THREADS + threadIdx.x; item < n_kv_heads * hd; item += gridDim.y * NR_THREADS) {
        const int h = item / hd, d = item - h * hd;
        const float value = d < vdim ? vrow[(size_t)h * vdim + d] : 0.f;
        vbase[(size_t)h * head_stride + (size_t)d * page_size] = from_float<T>(value);
    }
}

}  // namespace

extern "C" int mx_norm_rotate_kv_write(const float* proj, int ld, const int* positions, const float* freq, int rot,
                                       int interleaved, const float* q_weight, const float* k_weight, float eps,
                                       const int* slots, void* cache, long long n_pages, int page_size, void* q_out,
                                       int dtype, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, int hd,
                                       int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (hd < dim || hd < vdim) MX_REFUSE("attention operands: a padded head of %d holds neither %d nor %d", hd, dim, vdim);
    if (hd > 32 * NR_SLOTS) MX_REFUSE("attention operands: a head of %d entries (at most %d)", hd, 32 * NR_SLOTS);
    if (rot < 0 || rot % 2 != 0 || rot > dim) MX_REFUSE("attention operands: %d rotated entries in a head of %d", rot, dim);
    if (ld < (n_heads + n_kv_heads) * dim + n_kv_heads * vdim) MX_REFUSE("attention operands: projection rows are too short");
    const long long n_slots = n_pages * page_size;
    const int pieces = n_tokens >= 512 ? 1 : max(1, min(32, (n_heads + n_kv_heads + NR_WARPS - 1) / NR_WARPS));
    const dim3 grid(n_tokens, pieces);
    const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(norm_rotate_kv_write_kernel<float>, grid, dim3(NR_THREADS), smem, stream,
            proj, ld, positions, freq, rot, interleaved, q_weight, k_weight, eps, cache ? slots : nullptr, (float*)cache,
            n_slots, page_size, (float*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    else
        mx_launch_chained(norm_rotate_kv_write_kernel<__nv_bfloat16>, grid, dim3(NR_THREADS), smem, stream,
            proj, ld, positions, freq, rot, interleaved, q_weight, k_weight, eps, cache ? slots : nullptr,
            (__nv_bfloat16*)cache, n_slots, page_size, (__nv_bfloat16*)q_out, n_heads, n_kv_heads, dim, vdim, hd, status);
    return mx_launch_status();
}
