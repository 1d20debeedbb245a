// Tensor-core attention over the one-vector-per-token latent cache (bfloat16), for prompt portions and
// for decode tokens. Same mathematics and visibility rule as latent_attention.cu: every head of a token
// scores its latent-space query [rank | rot] against the cached vectors [latent | rotated part] of the
// positions it sees (j <= p and, with a window, j > p - window; a sink logit per head may join the denominator), softmax in float, and sums the first
// `rank` elements of those vectors.
//
// Rows. All heads share the keys, so the rows of a sequence are the (token, head) pairs, token-major:
// row r = t * heads + h. A block owns a tile of 64 consecutive rows and a split of the keys, walked in
// chunks of 32 positions; the rows of a tile sit on a few neighbouring tokens, so nearly every key a
// block loads is used by all of its rows.
//
// Work. Eight warps: warp = 2 * row group + half. A row group is 16 rows (an MMA M tile). Per chunk
// the two warps of a row group each compute the scores of 16 of the 32 keys over the whole key width
// (S = Q K^T, mma.sync.m16n8k16, bf16 in, float out), exchange row maxima and the rounded weights P
// through shared memory, and then each adds P V into its half of the `rank` value columns, which it
// keeps in registers (64 rows x 512 columns of float over 256 threads at the largest size). Keys reach
// shared memory with 16-byte cp.async copies, one chunk ahead of the arithmetic; positions outside the
// tile's range are zero-filled, never read. Row strides in shared memory are padded by 16 bytes so
// that ldmatrix rows fall into different banks.
// With more than one split a block writes unnormalised partials (max, sum, values) in the layout of
// attention.cu, whose merge kernel combines them.
#include <math.h>

#include "common.cuh"

extern "C" int mx_attention_merge_bf16_sink(const float* part_o, const float* part_ml, void* out, int out_stride,
                                            int n_tokens, int n_heads, int head_dim, int n_splits, const float* sink,
                                            cudaStream_t stream);

namespace {

constexpr int LT_ROWS = 64;
constexpr int LT_THREADS = 256;
constexpr int LT_KEYS = 32;
constexpr int LT_PSTRIDE = LT_KEYS + 8;      // row stride of the weights in shared memory (elements)

struct LatentMmaParams {
    const __nv_bfloat16* q;       // [tokens][heads][dk]
    const __nv_bfloat16* cache;   // [pages][page_size][dk]
    __nv_bfloat16* out;           // [tokens][heads][rank]
    float* part_o;                // [tokens][heads][splits][rank]
    float* part_ml;               // [tokens][heads][splits][2]
    const int* block_tables;
    const int* cu_q;
    const int* context_lens;
    const int* tiles;             // [n_tiles][2]: (sequence, first row); null: blockIdx.x is the sequence, .y the tile
    const float* sink;            // [heads] or null: exp(sink[h]) joins a row's denominator, with no value
    int* status;
    long long n_pages;
    int bt_stride, n_heads, rank, dk, page_size, window, n_splits;
    int q_rows;                   // rows of queries kept in shared memory: 64, or 16 when no tile has more (decoding)
    int stages;                   // key chunks in shared memory: 2, or 4 with q_rows = 16
    float scale;
};

__device__ __forceinline__ unsigned lt_smem(const void* ptr) { return (unsigned)__cvta_generic_to_shared(ptr); }

__device__ __forceinline__ void ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lt_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// NVT: value-column MMA tiles (8 columns each) a warp may keep; the launch picks the smallest that holds rank / 16.
template <int NVT>
__global__ void __launch_bounds__(LT_THREADS, 1)
latent_attention_mma_kernel(const LatentMmaParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = p.dk, rank = p.rank, heads = p.n_heads;
    const int ks = dk + 8;                                                    // padded row stride (elements)
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [q_rows][ks]
    __nv_bfloat16* k_s = q_s + p.q_rows * ks;                                 // [stages][32][ks]
    __nv_bfloat16* p_s = k_s + p.stages * LT_KEYS * ks;                       // [4][16][LT_PSTRIDE]
    float* red_max = reinterpret_cast<float*>(p_s + 4 * 16 * LT_PSTRIDE);     // [4][2][16]
    float* red_sum = red_max + 4 * 2 * 16;                                    // [4][2][16]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rg = warp >> 1, half = warp & 1;
    const int g = lane >> 2, tq = lane & 3;
    int seq, row0;
    if (p.tiles) { seq = p.tiles[2 * blockIdx.x]; row0 = p.tiles[2 * blockIdx.x + 1]; }
    else { seq = blockIdx.x; row0 = blockIdx.y * LT_ROWS; }
    const int split = blockIdx.z;
    pdl_trigger();
    pdl_wait();                           // the queries and this step's keys come from the kernels before
    const int t0 = p.cu_q[seq];
    const int n_rows = (p.cu_q[seq + 1] - t0) * heads;
    if (row0 >= n_rows) return;                                               // a sequence without tokens in this step
    const int rows_here = min(LT_ROWS, n_rows - row0);
    const int ctx = p.context_lens[seq];
    const int hi = ctx + (row0 + rows_here - 1) / heads;
    const int lo_tile = first_visible_key(ctx + row0 / heads, p.window);
    const int c_first = lo_tile / LT_KEYS, c_last = hi / LT_KEYS;
    const int per_split = (c_last - c_first + p.n_splits) / p.n_splits;
    const int c_begin = c_first + split * per_split;
    const int c_end = min(c_last + 1, c_begin + per_split);
    const size_t grow0 = (size_t)t0 * heads + row0;                           // first row of the tile among all rows

    // ---- the tile's queries
    const int vecs = dk >> 3;
    for (int item = tid; item < p.q_rows * vecs; item += LT_THREADS) {
        const int r = item / vecs, v = item - r * vecs;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < rows_here) val = *reinterpret_cast<const uint4*>(p.q + (grow0 + r) * dk + v * 8);
        *reinterpret_cast<uint4*>(q_s + r * ks + v * 8) = val;
    }

    const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
    // eight threads a key: one look at the block table per thread and chunk, then the key's vectors in turn
    auto issue = [&](int chunk, int stage) {
        const int j = tid >> 3, sub = tid & 7;
        const int kpos = chunk * LT_KEYS + j;
        __nv_bfloat16* d = k_s + (stage * LT_KEYS + j) * ks;
        const __nv_bfloat16* src = nullptr;
        if (kpos >= lo_tile && kpos <= hi) {
            const int lp = kpos / p.page_size;
            const long long page = lp < p.bt_stride ? bt[lp] : -1;
            if (page < 0 || page >= p.n_pages) {
                if (sub == 0) atomicOr(p.status, MX_STATUS_BAD_PAGE);
            } else {
                src = p.cache + ((size_t)page * p.page_size + (kpos - lp * p.page_size)) * dk;
            }
        }
        if (src) {
            for (int v = sub; v < vecs; v += 8) cp_async16(lt_smem(d + v * 8), src + v * 8);
        } else {
            for (int v = sub; v < vecs; v += 8) *reinterpret_cast<uint4*>(d + v * 8) = make_uint4(0, 0, 0, 0);
        }
    };

    // rows this thread holds in MMA accumulators: g and g + 8 of its row group
    int pos_r[2], lo_r[2];
    bool live_r[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = row0 + rg * 16 + g + 8 * e;
        live_r[e] = r < n_rows;
        pos_r[e] = ctx + r / heads;
        lo_r[e] = first_visible_key(pos_r[e], p.window);
    }
    float o[NVT][4];
#pragma unroll
    for (int n = 0; n < NVT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int nvp = rank >> 5;                       // pairs of value tiles a warp owns (rank / 2 columns)
    const bool rg_live = rg * 16 < rows_here;        // a row group beyond the tile's rows only helps with the copies
    const int col_base = half * (rank >> 1);

    // stages - 1 chunks are on their way while one is worked on (a group is committed every time, empty or
    // not, so that the count of groups to wait for never changes)
    const int ahead = p.stages - 1;
    for (int i = 0; i < ahead; ++i) {
        if (c_begin + i < c_end) issue(c_begin + i, i);
        cp_async_commit();
    }
    for (int chunk = c_begin; chunk < c_end; ++chunk) {
        const int stage = (chunk - c_begin) % p.stages;
        if (chunk + ahead < c_end) issue(chunk + ahead, (chunk - c_begin + ahead) % p.stages);
        cp_async_commit();
        if (ahead == 1) cp_async_wait<1>(); else cp_async_wait<3>();
        __syncthreads();                                                      // the chunk (and q_s) is in shared memory
        const __nv_bfloat16* kc = k_s + stage * LT_KEYS * ks;
        // ---- scores of this warp's 16 keys
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        if (rg_live) {
            // two chains of accumulators (even and odd steps of the contraction), added at the end: an MMA
            // need not wait for the one before it
            float s2[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s2[n][e] = 0.f;
            const unsigned a_addr = lt_smem(q_s + (rg * 16 + (lane & 15)) * ks + (lane >> 4) * 8);
            const unsigned b_addr = lt_smem(kc + (half * 16 + (lane >> 4) * 8 + (lane & 7)) * ks + ((lane >> 3) & 1) * 8);
            int kk = 0;
            for (; kk + 32 <= dk; kk += 32) {
                unsigned a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, d0, d1, d2, d3;
                ldsm_x4(a_addr + kk * 2, a0, a1, a2, a3);
                ldsm_x4(b_addr + kk * 2, b0, b1, b2, b3);
                ldsm_x4(a_addr + kk * 2 + 32, c0, c1, c2, c3);
                ldsm_x4(b_addr + kk * 2 + 32, d0, d1, d2, d3);
                lt_mma(s[0], a0, a1, a2, a3, b0, b1);
                lt_mma(s[1], a0, a1, a2, a3, b2, b3);
                lt_mma(s2[0], c0, c1, c2, c3, d0, d1);
                lt_mma(s2[1], c0, c1, c2, c3, d2, d3);
            }
            if (kk < dk) {
                unsigned a0, a1, a2, a3, b0, b1, b2, b3;
                ldsm_x4(a_addr + kk * 2, a0, a1, a2, a3);
                ldsm_x4(b_addr + kk * 2, b0, b1, b2, b3);
                lt_mma(s[0], a0, a1, a2, a3, b0, b1);
                lt_mma(s[1], a0, a1, a2, a3, b2, b3);
            }
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] += s2[n][e];
        }
        const int key0 = chunk * LT_KEYS + half * 16 + 2 * tq;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1, key = key0 + n * 8 + (e & 1);
                const bool seen = live_r[r] && key >= lo_r[r] && key <= pos_r[r];
                s[n][e] = seen ? s[n][e] * p.scale : -INFINITY;
                mx[r] = fmaxf(mx[r], s[n][e]);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            if (tq == 0) red_max[(rg * 2 + half) * 16 + g + 8 * r] = mx[r];
        }
        __syncthreads();
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float m_new = fmaxf(m_run[r], fmaxf(red_max[(rg * 2) * 16 + g + 8 * r],
                                                      red_max[(rg * 2 + 1) * 16 + g + 8 * r]));
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = __expf(m_run[r] - m_use);                              // 0 while nothing was seen before
            m_run[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const float w0 = __expf(s[n][2 * r] - m_use), w1 = __expf(s[n][2 * r + 1] - m_use);
                const __nv_bfloat162 packed = __floats2bfloat162_rn(w0, w1);
                // the sum is taken over the rounded weights, the ones the values are multiplied with
                sum += __low2float(packed) + __high2float(packed);
                *reinterpret_cast<__nv_bfloat162*>(p_s + (rg * 16 + g + 8 * r) * LT_PSTRIDE + half * 16 + n * 8 + 2 * tq) = packed;
            }
            l_run[r] = l_run[r] * alpha[r] + sum;
        }
        __syncthreads();
        // ---- O = alpha O + P V for this warp's columns
        if (rg_live) {
#pragma unroll
            for (int n = 0; n < NVT; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            const unsigned pa_addr = lt_smem(p_s + (rg * 16 + (lane & 15)) * LT_PSTRIDE + (lane >> 4) * 8);
            unsigned pa[2][4];
            ldsm_x4(pa_addr, pa[0][0], pa[0][1], pa[0][2], pa[0][3]);
            ldsm_x4(pa_addr + 32, pa[1][0], pa[1][1], pa[1][2], pa[1][3]);
            // value tiles: matrices (keys 0-7 | 8-15) x (columns 0-7 | 8-15) of each pair of tiles, transposed on load
            const unsigned v_addr = lt_smem(kc + (((lane >> 3) & 1) * 8 + (lane & 7)) * ks + col_base + (lane >> 4) * 8);
#pragma unroll
            for (int jp = 0; jp < NVT / 2; ++jp) {
                if (jp < nvp) {
#pragma unroll
                    for (int kstep = 0; kstep < 2; ++kstep) {
                        unsigned b0, b1, b2, b3;
                        ldsm_x4_trans(v_addr + (kstep * 16 * ks + jp * 16) * 2, b0, b1, b2, b3);
                        lt_mma(o[2 * jp], pa[kstep][0], pa[kstep][1], pa[kstep][2], pa[kstep][3], b0, b1);
                        lt_mma(o[2 * jp + 1], pa[kstep][0], pa[kstep][1], pa[kstep][2], pa[kstep][3], b2, b3);
                    }
                }
            }
        }
        __syncthreads();                                                      // stage, weights and maxima may be overwritten
    }
    cp_async_wait<0>();

    // ---- the rows' sums: over the quad, then over the two halves of the keys
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        if (tq == 0) red_sum[(rg * 2 + half) * 16 + g + 8 * r] = l_run[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!live_r[r]) continue;
        const float l = red_sum[(rg * 2) * 16 + g + 8 * r] + red_sum[(rg * 2 + 1) * 16 + g + 8 * r];
        const size_t grow = grow0 + rg * 16 + g + 8 * r;
        if (p.n_splits == 1) {
            // the sink counts once (with key splits the merge kernel adds it)
            const float extra = p.sink ? __expf(p.sink[(int)(grow % heads)] - m_run[r]) : 0.f;
            const float inv = 1.f / (l + extra);
            __nv_bfloat16* dst = p.out + grow * rank + col_base + 2 * tq;
#pragma unroll
            for (int n = 0; n < NVT; ++n)
                if (n < 2 * nvp)
                    *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        } else {
            const size_t base = grow * p.n_splits + split;
            float* dst = p.part_o + base * rank + col_base + 2 * tq;
#pragma unroll
            for (int n = 0; n < NVT; ++n)
                if (n < 2 * nvp) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            if (half == 0 && tq == 0) { p.part_ml[base * 2] = m_run[r]; p.part_ml[base * 2 + 1] = l; }
        }
    }
}

template <int NVT>
int launch_latent_mma(const LatentMmaParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    cudaFuncSetAttribute(latent_attention_mma_kernel<NVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mx_launch_chained(latent_attention_mma_kernel<NVT>, grid, dim3(LT_THREADS), smem, stream, p);
    return mx_launch_status();
}

}  // namespace

static size_t latent_mma_smem(int dk, int q_rows, int stages) {
    return (size_t)(q_rows + stages * LT_KEYS) * (dk + 8) * 2 + 4 * 16 * LT_PSTRIDE * 2 + 2 * 4 * 2 * 16 * 4;
}

extern "C" int mx_latent_attention_mma_supported(int rank, int dk) {
    const size_t smem = latent_mma_smem(dk, LT_ROWS, 2);
    return rank > 0 && rank % 32 == 0 && rank <= 512 && dk >= rank && dk % 16 == 0 && smem <= 220 * 1024;
}

// few_rows != 0: every tile has at most 16 rows (see below).
// tiles: [n_tiles][2] (sequence, first row) with grid_y = 1, or null with one block row per sequence and
// grid_y row tiles per sequence (a fixed-size batch of decoding requests). scratch: float,
// mx_attention_scratch_bytes(n_tokens, n_heads, rank, n_splits) bytes when n_splits > 1.
extern "C" int mx_latent_attention_mma(const void* q, const void* cache, long long n_pages, int page_size,
                                       const int* block_tables, int bt_stride, const int* cu_q,
                                       const int* context_lens, const int* tiles, int n_tiles, int grid_y,
                                       int n_tokens, int n_heads, int rank, int dk, int window, float scale,
                                       void* out, int n_splits, float* scratch, int few_rows, const float* sink,
                                       int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || n_tiles <= 0) return MX_OK;
    if (!mx_latent_attention_mma_supported(rank, dk))
        MX_REFUSE("tensor-core latent attention: rank %d of a key of %d is not taken", rank, dk);
    if (n_splits < 1 || (n_splits > 1 && scratch == nullptr)) MX_REFUSE("latent attention: %d splits without scratch", n_splits);
    LatentMmaParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * rank : nullptr;
    p.block_tables = block_tables; p.cu_q = cu_q; p.context_lens = context_lens; p.tiles = tiles; p.sink = sink;
    p.status = status; p.n_pages = n_pages; p.bt_stride = bt_stride; p.n_heads = n_heads; p.rank = rank;
    p.dk = dk; p.page_size = page_size; p.window = window; p.n_splits = n_splits; p.scale = scale;
    // few_rows: the caller vouches that no tile has more than 16 rows (single tokens of at most 16 heads); the
    // room of the other 48 query rows then goes to two more key chunks in flight
    p.q_rows = few_rows ? 16 : LT_ROWS;
    p.stages = (few_rows && latent_mma_smem(dk, 16, 4) <= 220 * 1024) ? 4 : 2;
    const size_t smem = latent_mma_smem(dk, p.q_rows, p.stages);
    dim3 grid(n_tiles, tiles ? 1 : grid_y, n_splits);
    int rc;
    if (rank <= 128) rc = launch_latent_mma<8>(p, grid, smem, stream);
    else if (rank <= 256) rc = launch_latent_mma<16>(p, grid, smem, stream);
    else rc = launch_latent_mma<32>(p, grid, smem, stream);
    if (rc != MX_OK || n_splits == 1) return rc;
    return mx_attention_merge_bf16_sink(p.part_o, p.part_ml, out, n_heads * rank, n_tokens, n_heads, rank, n_splits, sink,
                                        stream);
}
