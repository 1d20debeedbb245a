// Attention over a cache of one shared latent vector per token (multi-head latent attention in its
// "absorbed" form), with an optional sliding window.
//
// Per token the cache holds ONE vector of Dk = rank + rot elements for all heads: the normalised
// latent c (rank) followed by a rotated key part r (rot). With the per-head key expansion folded
// into the query (q' = Uk_h^T q_plain, done by a batched product before this kernel), head h's score
// against token j is (q'_h . c_j + q_rot_h . r_j) * scale, and its output in latent space is
// sum_j p_j c_j; the per-head value expansion Uv_h follows as another batched product. So this is
// attention with one key/value head whose value is the first `rank` elements of its key.
//
// mx_latent_prepare (per token one block for the cache vector and one per four query heads) reads the float result of the fused query / down
// projection, [q heads (plain | rot) | latent | shared rot], and writes
//   q_plain [tokens][heads * dim]          (activation dtype: the batched product's operand)
//   q_lat   [tokens][heads][Dk]            the rotated query part at offset rank
//   cache   [slot][Dk]                     unit(latent) * weight, then the rotated shared part
// (the latent and the shared part may also come from rows of their own, `kvd`).
// Rotation: of the `rot` elements the first rot_dims are rotated, pair (i, i + rot_dims/2) or, `interleaved`, (2i, 2i + 1), by the
// angle position * freq[i] (float), cos and sin times `amplitude`; the rest pass unchanged.
//
// mx_latent_attention: one block per (token, group of up to LAT_HEADS heads). Keys are walked in
// chunks of 32 positions (one key per lane) from max(0, p - window + 1) to p; scores, the running
// softmax and the weighted sum are float. A query at position p sees key j iff j <= p and
// (window == 0 or j > p - window; window < 0: j in the query's own block of -window positions). A sink (one
// logit per head, or none) joins the softmax's denominator without a value.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LAT_THREADS = 128;
constexpr int LAT_WARPS = LAT_THREADS / 32;
constexpr int LAT_HEADS = 8;      // heads per block at most
constexpr int LAT_KEYS = 32;
constexpr int LAT_PREP_HEADS = 4;  // query heads per block of the preparing kernel

// Entry d of a vector whose first rot_dims entries are rotated: pair i is (i, i + half) or, interleaved,
// (2i, 2i + 1); cs holds cos[half] then sin[half] of the pairs' angles.
__device__ __forceinline__ float rotated_entry(const float* src, int d, int half, int rot_dims, int interleaved,
                                               const float* cs) {
    if (d >= rot_dims) return src[d];
    if (interleaved) {
        const int i = d >> 1;
        return (d & 1) ? src[d] * cs[i] + src[d - 1] * cs[half + i] : src[d] * cs[i] - src[d + 1] * cs[half + i];
    }
    if (d < half) return src[d] * cs[d] - src[d + half] * cs[half + d];
    return src[d] * cs[d - half] + src[d - half] * cs[d];
}

template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prepare_kernel(const float* __restrict__ qd, int ld, const float* __restrict__ kvd, int ld_kv, int interleaved,
                      const int* __restrict__ positions,
                      const float* __restrict__ freq, float amplitude, const float* __restrict__ latent_weight,
                      float eps, const int* __restrict__ slots, T* __restrict__ cache, long long n_slots,
                      T* __restrict__ q_plain, T* __restrict__ q_lat, int n_heads, int dim, int rot,
                      int rot_dims, int rank, int* status) {
    extern __shared__ float cs[];               // cos[half], sin[half]
    __shared__ float scratch[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot_dims >> 1;
    const int dk = rank + rot;
    const float pos = (float)positions[t];      // step metadata and constants: no kernel writes them
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = pos * freq[i];
        cs[i] = cosf(angle) * amplitude;
        cs[half + i] = sinf(angle) * amplitude;
    }
    __syncthreads();
    pdl_wait();
    const float* row = after_wait(qd) + (size_t)t * ld;
    const int qw = dim + rot;
    if (blockIdx.y > 0) {
        // blocks 1 .. of a token: LAT_PREP_HEADS query heads each
        const int h0 = (blockIdx.y - 1) * LAT_PREP_HEADS, h1 = min(n_heads, h0 + LAT_PREP_HEADS);
        for (int h = h0; h < h1; ++h) {
            const float* src = row + (size_t)h * qw;
            // the plain part, as the batched product's operand
            for (int d = threadIdx.x; d < dim; d += blockDim.x)
                q_plain[((size_t)t * n_heads + h) * dim + d] = from_float<T>(src[d]);
            // the rotated part, to the tail of the head's latent-space query
            src += dim;
            for (int d = threadIdx.x; d < rot; d += blockDim.x) {
                const float v = rotated_entry(src, d, half, rot_dims, interleaved, cs);
                q_lat[((size_t)t * n_heads + h) * dk + rank + d] = from_float<T>(v);
            }
        }
        return;
    }
    // block 0 of a token: its cache vector
    const long long slot = slots ? slots[t] : -1;
    // the latent and the shared rotated part follow the query heads, or lie in rows of their own
    const float* lat = kvd ? after_wait(kvd) + (size_t)t * ld_kv : row + (size_t)n_heads * qw;
    float s = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) s = fmaf(lat[i], lat[i], s);
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)rank + eps);
    if (slot == -1) return;                     // a padding row, or a reader of somebody else's cache
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
        return;
    }
    T* dst = cache + (size_t)slot * dk;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(lat[i] * inv * latent_weight[i]);
    const float* src = lat + rank;
    for (int d = threadIdx.x; d < rot; d += blockDim.x) {
        const float v = rotated_entry(src, d, half, rot_dims, interleaved, cs);
        dst[rank + d] = from_float<T>(v);
    }
}

struct LatentParams {
    const void* q;            // [tokens][heads][dk]
    const void* cache;        // [pages][page_size][dk]
    void* out;                // [tokens][heads][rank]
    const int* block_tables;
    const int* tok_seq;
    const int* positions;
    const float* sink;        // [n_heads] or null: exp(sink[h]) joins the softmax's denominator, with no value
    int* status;
    long long n_pages;
    int bt_stride, n_heads, rank, dk, page_size, window;
    float scale;
};

template <typename T, int SLOTS>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const LatentParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = p.dk, rank = p.rank;
    const int kst = dk + 1;                                   // row stride of the staged keys (odd: no conflicts)
    float* q_s = reinterpret_cast<float*>(smem_raw);          // [LAT_HEADS][dk]
    float* k_s = q_s + LAT_HEADS * dk;                        // [LAT_KEYS][kst]
    float* p_s = k_s + LAT_KEYS * kst;                        // [LAT_HEADS][LAT_KEYS]
    float* alpha_s = p_s + LAT_HEADS * LAT_KEYS;              // [LAT_HEADS]
    float* l_s = alpha_s + LAT_HEADS;                         // [LAT_HEADS]

    const int t = blockIdx.x;
    const int head0 = blockIdx.y * LAT_HEADS;
    const int gc = min(LAT_HEADS, p.n_heads - head0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    T* orow = reinterpret_cast<T*>(p.out) + ((size_t)t * p.n_heads + head0) * rank;
    const int seq = p.tok_seq[t];
    if (seq < 0) {                                            // a padding row of a fixed-size batch
        for (int i = tid; i < gc * rank; i += LAT_THREADS) orow[i] = from_float<T>(0.f);
        return;
    }
    const int pos = p.positions[t];
    const int lo = first_visible_key(pos, p.window);
    const T* qrow = reinterpret_cast<const T*>(p.q) + ((size_t)t * p.n_heads + head0) * dk;
    for (int i = tid; i < gc * dk; i += LAT_THREADS) q_s[i] = to_float(qrow[i]) * p.scale;

    float acc[LAT_HEADS][SLOTS];
#pragma unroll
    for (int h = 0; h < LAT_HEADS; ++h)
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) acc[h][s] = 0.f;
    constexpr int HPW = LAT_HEADS / LAT_WARPS;                // heads whose softmax a warp keeps
    float m_run[HPW], l_run[HPW];
#pragma unroll
    for (int hs = 0; hs < HPW; ++hs) { m_run[hs] = -INFINITY; l_run[hs] = 0.f; }

    const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
    const T* cache = reinterpret_cast<const T*>(p.cache);
    for (int c0 = (lo / LAT_KEYS) * LAT_KEYS; c0 <= pos; c0 += LAT_KEYS) {
        __syncthreads();                                      // the chunk before is used up (and q_s is written)
        for (int item = tid; item < LAT_KEYS * dk; item += LAT_THREADS) {
            const int j = item / dk, d = item - j * dk;
            const int kpos = c0 + j;
            float v = 0.f;
            if (kpos >= lo && kpos <= pos) {
                const int lp = kpos / p.page_size;
                const long long page = (lp < p.bt_stride) ? bt[lp] : -1;
                if (page < 0 || page >= p.n_pages) {
                    if (d == 0) atomicOr(p.status, MX_STATUS_BAD_PAGE);
                } else {
                    v = to_float(cache[((size_t)page * p.page_size + (kpos - lp * p.page_size)) * dk + d]);
                }
            }
            k_s[j * kst + d] = v;
        }
        __syncthreads();
        {
            const int kpos = c0 + lane;
            const bool valid = kpos >= lo && kpos <= pos;
            const float* kr = k_s + lane * kst;
#pragma unroll
            for (int hs = 0; hs < HPW; ++hs) {
                const int h = warp + hs * LAT_WARPS;
                if (h >= gc) continue;
                const float* qh = q_s + h * dk;
                float s = 0.f;
                for (int d = 0; d < dk; ++d) s = fmaf(qh[d], kr[d], s);
                s = valid ? s : -INFINITY;
                const float m_new = fmaxf(m_run[hs], warp_max(s));      // finite: the chunk holds a visible key
                const float w = valid ? expf(s - m_new) : 0.f;
                const float a = expf(m_run[hs] - m_new);                // 0 at the first chunk
                l_run[hs] = l_run[hs] * a + warp_sum(w);
                m_run[hs] = m_new;
                p_s[h * LAT_KEYS + lane] = w;
                if (lane == 0) alpha_s[h] = a;
            }
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int d = tid + s * LAT_THREADS;
            if (d >= rank) break;
#pragma unroll
            for (int h = 0; h < LAT_HEADS; ++h) {
                if (h >= gc) break;
                float a = acc[h][s] * alpha_s[h];
                const float* ph = p_s + h * LAT_KEYS;
#pragma unroll 8
                for (int j = 0; j < LAT_KEYS; ++j) a = fmaf(ph[j], k_s[j * kst + d], a);
                acc[h][s] = a;
            }
        }
    }
#pragma unroll
    for (int hs = 0; hs < HPW; ++hs) {
        const int h = warp + hs * LAT_WARPS;
        // the sink counts once in the denominator and brings no value
        if (h < gc && lane == 0) l_s[h] = l_run[hs] + (p.sink ? expf(p.sink[head0 + h] - m_run[hs]) : 0.f);
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int d = tid + s * LAT_THREADS;
        if (d >= rank) break;
#pragma unroll
        for (int h = 0; h < LAT_HEADS; ++h) {
            if (h >= gc) break;
            orow[(size_t)h * rank + d] = from_float<T>(acc[h][s] / l_s[h]);
        }
    }
}

template <typename T, int SLOTS>
int launch_latent(const LatentParams& p, int n_tokens, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(latent_attention_kernel<T, SLOTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(n_tokens, (p.n_heads + LAT_HEADS - 1) / LAT_HEADS);
    latent_attention_kernel<T, SLOTS><<<grid, LAT_THREADS, smem, stream>>>(p);
    return mx_launch_status();
}

}  // namespace

extern "C" int mx_latent_prepare(const float* qd, int ld, const float* kvd, int ld_kv, int interleaved, const int* positions, const float* freq,
                                 float amplitude, const float* latent_weight, float eps, const int* slots,
                                 void* cache, long long n_pages, int page_size, void* q_plain, void* q_lat,
                                 int dtype, int n_tokens, int n_heads, int dim, int rot, int rot_dims, int rank,
                                 int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1))
        MX_REFUSE("latent attention: %d rotated dimensions of %d", rot_dims, rot);
    if (ld < n_heads * (dim + rot) + (kvd ? 0 : rank + rot) || (kvd && ld_kv < rank + rot)) MX_REFUSE("latent attention: projection rows are too short");
    const size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 1) * sizeof(float);
    const long long n_slots = n_pages * page_size;
    const dim3 grid(n_tokens, 1 + (n_heads + LAT_PREP_HEADS - 1) / LAT_PREP_HEADS);
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(latent_prepare_kernel<float>, grid, dim3(LAT_THREADS), smem, stream,
            qd, ld, kvd, ld_kv, interleaved, positions, freq, amplitude, latent_weight, eps, cache ? slots : nullptr, (float*)cache, n_slots,
            (float*)q_plain, (float*)q_lat, n_heads, dim, rot, rot_dims, rank, status);
    else
        mx_launch_chained(latent_prepare_kernel<__nv_bfloat16>, grid, dim3(LAT_THREADS), smem, stream,
            qd, ld, kvd, ld_kv, interleaved, positions, freq, amplitude, latent_weight, eps, cache ? slots : nullptr, (__nv_bfloat16*)cache,
            n_slots, (__nv_bfloat16*)q_plain, (__nv_bfloat16*)q_lat, n_heads, dim, rot, rot_dims, rank, status);
    return mx_launch_status();
}

extern "C" int mx_latent_attention(const void* q, const void* cache, int dtype, long long n_pages, int page_size,
                                   const int* block_tables, int bt_stride, const int* tok_seq,
                                   const int* positions, int n_tokens, int n_heads, int rank, int dk, int window,
                                   float scale, void* out, const float* sink, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (rank <= 0 || dk < rank) MX_REFUSE("latent attention: rank %d of a key of %d", rank, dk);
    if (rank > 8 * LAT_THREADS) MX_REFUSE("latent attention: a latent of %d exceeds %d", rank, 8 * LAT_THREADS);
    LatentParams p;
    p.q = q; p.cache = cache; p.out = out; p.block_tables = block_tables; p.tok_seq = tok_seq;
    p.positions = positions; p.sink = sink; p.status = status; p.n_pages = n_pages; p.bt_stride = bt_stride;
    p.n_heads = n_heads; p.rank = rank; p.dk = dk; p.page_size = page_size; p.window = window; p.scale = scale;
    const size_t smem = sizeof(float) * ((size_t)LAT_HEADS * dk + (size_t)LAT_KEYS * (dk + 1) +
                                         LAT_HEADS * LAT_KEYS + 2 * LAT_HEADS);
    if (smem > 200 * 1024) MX_REFUSE("latent attention: a key of %d elements does not fit in shared memory", dk);
    const int slots = (rank + LAT_THREADS - 1) / LAT_THREADS;
#define MX_LAT(T)                                                       \
    (slots <= 1 ? launch_latent<T, 1>(p, n_tokens, smem, stream)        \
     : slots <= 2 ? launch_latent<T, 2>(p, n_tokens, smem, stream)      \
     : slots <= 4 ? launch_latent<T, 4>(p, n_tokens, smem, stream)      \
                  : launch_latent<T, 8>(p, n_tokens, smem, stream))
    return dtype == MX_DTYPE_F32 ? MX_LAT(float) : MX_LAT(__nv_bfloat16);
#undef MX_LAT
}
