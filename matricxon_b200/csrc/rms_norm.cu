// RMS norm over rows of the float residual stream, and the post-norm step that forms its own input.
//
//   unit(x) = x / sqrt(mean(x^2) + eps)          (eps inside the root)
//   mx_rmsnorm:      out[r] = unit(x[rows ? rows[r] : r]) * (offset + weight)      (rows of x `x_stride` floats apart)
//   mx_rmsnorm_branch_add: x[r] <- x[r] + unit(y[r]) * wb      (in place, float: a branch normalised on its way in)
//                    out[r] <- unit(x[r]) * wn in the activation dtype (the next sublayer's normalised input;
//                    wn null: x[r] itself, rounded; out null: nothing)
//   mx_rmsnorm_sum:  x[r]  <- unit(alpha * x[r] + acc[r]) * (offset + weight)   (in place, float)
//                    act[r] <- the same row rounded to the activation dtype (optional)
//
// `offset` is 1 for checkpoints that store the scale as its distance from one and 0 for a plain
// scale. The second form is a post-norm sublayer's end: `acc` is the float result of the sublayer's
// last product, `alpha` the weight of the skip path; the next sublayer reads `act` (a bfloat16 copy
// when serving; on the 32-bit path it reads x itself and act is null).
//
// The float4 form of the post-norm sum takes part in chained launches (programmatic dependent launch).
// One block per row; sums of squares are float and their order depends on the thread layout alone,
// so a row's result does not depend on the other rows of the step.
// mx_cast_rows rounds a float matrix to the activation dtype (the first sublayer's input).
#include "common.cuh"

namespace {

constexpr int RMS_MAX_PER_THREAD = 16;   // row values a thread keeps in registers

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 packed;
    packed.x = *reinterpret_cast<unsigned*>(&lo);
    packed.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const float* __restrict__ weight, float offset, TOut* __restrict__ out,
                               int hidden, float eps, long long x_stride) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * x_stride;
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        s = fmaf(v, v, s);
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    TOut* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = from_float<TOut>(xr[i] * inv * (offset + weight[i]));
}

template <typename TAct>
__global__ void rmsnorm_sum_kernel(float* x, const float* __restrict__ acc, float alpha,
                                   const float* __restrict__ weight, float offset, TAct* act,
                                   int hidden, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * hidden;
    const float* ar = acc + (size_t)r * hidden;
    float kept[RMS_MAX_PER_THREAD];
    float s = 0.f;
    int n = 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n) {
        const float v = fmaf(alpha, xr[i], ar[i]);
        if (n < RMS_MAX_PER_THREAD) kept[n] = v; else xr[i] = v;      // long rows park the sum in x itself
        s = fmaf(v, v, s);
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    n = 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n) {
        const float v = (n < RMS_MAX_PER_THREAD ? kept[n] : xr[i]) * inv * (offset + weight[i]);
        xr[i] = v;
        if (act) act[(size_t)r * hidden + i] = from_float<TAct>(v);
    }
}

// The same for rows whose length is a multiple of 4: float4 accesses, up to RMS_VEC float4 a thread in registers.
constexpr int RMS_VEC = 4;

template <typename TAct>
__global__ void rmsnorm_sum_vec_kernel(float* x, const float* __restrict__ acc, float alpha,
                                       const float* __restrict__ weight, float offset, TAct* act, int hidden,
                                       float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    x = after_wait(x);
    acc = after_wait(acc);
    const int r = blockIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * hidden);
    const float4* ar = reinterpret_cast<const float4*>(acc + (size_t)r * hidden);
    const float4* wr = reinterpret_cast<const float4*>(weight);
    const int vecs = hidden >> 2;
    float4 kept[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            const float4 a = xr[i], b = ar[i];
            kept[n] = make_float4(fmaf(alpha, a.x, b.x), fmaf(alpha, a.y, b.y), fmaf(alpha, a.z, b.z), fmaf(alpha, a.w, b.w));
            s = fmaf(kept[n].x, kept[n].x, s); s = fmaf(kept[n].y, kept[n].y, s);
            s = fmaf(kept[n].z, kept[n].z, s); s = fmaf(kept[n].w, kept[n].w, s);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            const float4 w = wr[i];
            const float4 v = make_float4(kept[n].x * inv * (offset + w.x), kept[n].y * inv * (offset + w.y),
                                         kept[n].z * inv * (offset + w.z), kept[n].w * inv * (offset + w.w));
            xr[i] = v;
            if (act) {
                TAct* dst = act + (size_t)r * hidden + 4 * i;
                dst[0] = from_float<TAct>(v.x); dst[1] = from_float<TAct>(v.y);
                dst[2] = from_float<TAct>(v.z); dst[3] = from_float<TAct>(v.w);
            }
        }
    }
}

// x += unit(y) * wb, then out = unit(x) * wn (or x, or nothing): one block per row, both rows in registers
// (longer rows are read again), float statistics in an order that the thread layout alone fixes.
template <typename TAct>
__global__ void rmsnorm_branch_add_kernel(float* x, const float* y, const float* __restrict__ wb,
                                          const float* __restrict__ wn, TAct* out, int hidden, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    x = after_wait(x);
    y = after_wait(y);
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * hidden;
    const float* yr = y + (size_t)r * hidden;
    float kept[RMS_MAX_PER_THREAD];
    float s = 0.f;
    int n = 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n) {
        const float v = yr[i];
        if (n < RMS_MAX_PER_THREAD) kept[n] = v;
        s = fmaf(v, v, s);
    }
    const float inv_y = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    s = 0.f;
    n = 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n) {
        const float b = n < RMS_MAX_PER_THREAD ? kept[n] : yr[i];
        const float v = xr[i] + b * inv_y * wb[i];
        xr[i] = v;
        if (n < RMS_MAX_PER_THREAD) kept[n] = v;
        s = fmaf(v, v, s);
    }
    if (out == nullptr) return;
    TAct* o = out + (size_t)r * hidden;
    if (wn == nullptr) {
        n = 0;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n)
            o[i] = from_float<TAct>(n < RMS_MAX_PER_THREAD ? kept[n] : xr[i]);
        return;
    }
    const float inv_x = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    n = 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x, ++n)
        o[i] = from_float<TAct>((n < RMS_MAX_PER_THREAD ? kept[n] : xr[i]) * inv_x * wn[i]);
}

// The float4 forms of the two kernels above, for rows whose length (and stride) is a multiple of 4 and that fit in
// RMS_VEC float4 a thread: one trip to memory for the row, which stays in registers between the passes. Few rows
// (a decode step) get a thread per float4, so that the row's latency is all there is.
template <typename TOut>
__global__ void rmsnorm_vec_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ weight,
                                   float offset, TOut* __restrict__ out, int hidden, float eps, long long x_stride) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int vecs = hidden >> 2;
    const float4* wr = reinterpret_cast<const float4*>(weight);
    float4 w[RMS_VEC];
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {                       // the weight does not depend on the kernel before
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) w[n] = wr[i];
    }
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(after_wait(x) + (size_t)(rows ? rows[r] : r) * x_stride);
    float4 kept[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            kept[n] = xr[i];
            s = fmaf(kept[n].x, kept[n].x, s); s = fmaf(kept[n].y, kept[n].y, s);
            s = fmaf(kept[n].z, kept[n].z, s); s = fmaf(kept[n].w, kept[n].w, s);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            TOut* dst = out + (size_t)r * hidden + 4 * i;
            store4(dst, kept[n].x * inv * (offset + w[n].x), kept[n].y * inv * (offset + w[n].y),
                   kept[n].z * inv * (offset + w[n].z), kept[n].w * inv * (offset + w[n].w));
        }
    }
}

template <typename TAct>
__global__ void rmsnorm_branch_add_vec_kernel(float* x, const float* y, const float* __restrict__ wb,
                                              const float* __restrict__ wn, TAct* out, int hidden, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    x = after_wait(x);
    y = after_wait(y);
    const int r = blockIdx.x;
    const int vecs = hidden >> 2;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * hidden);
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * hidden);
    float4 branch[RMS_VEC], row[RMS_VEC];
    float s = 0.f;
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            branch[n] = yr[i];
            row[n] = xr[i];
            s = fmaf(branch[n].x, branch[n].x, s); s = fmaf(branch[n].y, branch[n].y, s);
            s = fmaf(branch[n].z, branch[n].z, s); s = fmaf(branch[n].w, branch[n].w, s);
        }
    }
    const float inv_y = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    s = 0.f;
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            const float4 w = reinterpret_cast<const float4*>(wb)[i];
            row[n] = make_float4(row[n].x + branch[n].x * inv_y * w.x, row[n].y + branch[n].y * inv_y * w.y,
                                 row[n].z + branch[n].z * inv_y * w.z, row[n].w + branch[n].w * inv_y * w.w);
            xr[i] = row[n];
            s = fmaf(row[n].x, row[n].x, s); s = fmaf(row[n].y, row[n].y, s);
            s = fmaf(row[n].z, row[n].z, s); s = fmaf(row[n].w, row[n].w, s);
        }
    }
    if (out == nullptr) return;
    float inv_x = 1.f;
    if (wn != nullptr) inv_x = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
#pragma unroll
    for (int n = 0; n < RMS_VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < vecs) {
            float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
            if (wn != nullptr) w = reinterpret_cast<const float4*>(wn)[i];
            store4(out + (size_t)r * hidden + 4 * i, row[n].x * inv_x * w.x, row[n].y * inv_x * w.y,
                   row[n].z * inv_x * w.z, row[n].w * inv_x * w.w);
        }
    }
}

// Threads a row for the float4 kernels, or 0 when the row does not fit: a thread per float4 for few rows.
int vec_threads_for(int n_rows, int hidden) {
    if (hidden % 4 != 0) return 0;
    const int vecs = hidden / 4;
    int threads = n_rows <= 64 ? (vecs + 31) / 32 * 32 : (vecs >= 1024 ? 512 : 256);
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    return (long long)threads * RMS_VEC >= vecs ? threads : 0;
}

__global__ void cast_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __float2bfloat16_rn(x[i]);
}

int threads_for(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128); }

}  // namespace

extern "C" int mx_rmsnorm(const float* x, const int* rows, const float* weight, float offset, void* out,
                          int out_dtype, int n_rows, int hidden, float eps, long long x_stride, cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (hidden <= 0) MX_REFUSE("rmsnorm: hidden must be positive, got %d", hidden);
    const int vec_threads = (x_stride % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) ? vec_threads_for(n_rows, hidden) : 0;
    if (vec_threads > 0) {
        if (out_dtype == MX_DTYPE_F32)
            mx_launch_chained(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(vec_threads), 0, stream, x, rows, weight,
                              offset, (float*)out, hidden, eps, x_stride);
        else
            mx_launch_chained(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vec_threads), 0, stream, x, rows,
                              weight, offset, (__nv_bfloat16*)out, hidden, eps, x_stride);
        return mx_launch_status();
    }
    const int threads = threads_for(hidden);
    if (out_dtype == MX_DTYPE_F32)
        rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>(x, rows, weight, offset, (float*)out, hidden, eps, x_stride);
    else
        rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(x, rows, weight, offset,
                                                                     (__nv_bfloat16*)out, hidden, eps, x_stride);
    return mx_launch_status();
}

extern "C" int mx_rmsnorm_branch_add(float* x, const float* y, const float* wb, const float* wn, void* out,
                                     int out_dtype, int n_rows, int hidden, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (hidden <= 0) MX_REFUSE("rmsnorm: hidden must be positive, got %d", hidden);
    const int vec_threads = vec_threads_for(n_rows, hidden);
    if (vec_threads > 0) {
        if (out_dtype == MX_DTYPE_F32)
            mx_launch_chained(rmsnorm_branch_add_vec_kernel<float>, dim3(n_rows), dim3(vec_threads), 0, stream, x, y, wb,
                              wn, (float*)out, hidden, eps);
        else
            mx_launch_chained(rmsnorm_branch_add_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vec_threads), 0, stream, x,
                              y, wb, wn, (__nv_bfloat16*)out, hidden, eps);
        return mx_launch_status();
    }
    // few rows (a decode step): the row's latency is all there is, so more threads a row
    const int threads = n_rows <= 64 ? min(1024, max(128, (hidden + 127) / 128 * 32)) : threads_for(hidden);
    if (out_dtype == MX_DTYPE_F32)
        mx_launch_chained(rmsnorm_branch_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, wb, wn,
                          (float*)out, hidden, eps);
    else
        mx_launch_chained(rmsnorm_branch_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, y, wb,
                          wn, (__nv_bfloat16*)out, hidden, eps);
    return mx_launch_status();
}

extern "C" int mx_rmsnorm_sum(float* x, const float* acc, float alpha, const float* weight, float offset,
                              void* act, int act_dtype, int n_rows, int hidden, float eps,
                              cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (hidden <= 0) MX_REFUSE("rmsnorm: hidden must be positive, got %d", hidden);
    if (acc == nullptr) MX_REFUSE("rmsnorm with sum: no accumulator");
    if (hidden % 4 == 0 && hidden <= 4 * RMS_VEC * 1024) {
        // a thread per float4 where the row allows it (few rows: the row's latency is all there is); long rows
        // take up to RMS_VEC float4 a thread
        int vthreads = ((hidden / 4 + RMS_VEC - 1) / RMS_VEC + 31) / 32 * 32;
        if (n_rows <= 64) vthreads = (hidden / 4 + 31) / 32 * 32;
        vthreads = vthreads > 1024 ? 1024 : vthreads;
        if (act == nullptr || act_dtype == MX_DTYPE_F32)
            mx_launch_chained(rmsnorm_sum_vec_kernel<float>, dim3(n_rows), dim3(vthreads), 0, stream, x, acc, alpha,
                              weight, offset, (float*)act, hidden, eps);
        else
            mx_launch_chained(rmsnorm_sum_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vthreads), 0, stream, x, acc,
                              alpha, weight, offset, (__nv_bfloat16*)act, hidden, eps);
        return mx_launch_status();
    }
    const int threads = threads_for(hidden);
    if (act == nullptr || act_dtype == MX_DTYPE_F32)
        rmsnorm_sum_kernel<float><<<n_rows, threads, 0, stream>>>(x, acc, alpha, weight, offset, (float*)act,
                                                                 hidden, eps);
    else
        rmsnorm_sum_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(x, acc, alpha, weight, offset,
                                                                         (__nv_bfloat16*)act, hidden, eps);
    return mx_launch_status();
}

extern "C" int mx_cast_rows(const float* x, void* out, long long count, cudaStream_t stream) {
    if (count <= 0) return MX_OK;
    cast_rows_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(x, (__nv_bfloat16*)out, count);
    return mx_launch_status();
}
