// Latent attention, the parts around the products, for any sizes in 32-bit arithmetic.
//
// The cache holds one row per token, [latent c (rank) | rotated key part (rot)], in pages [pages, page_size, rank + rot];
// every head reads the same rows. Queries arrive folded: [a_h (rank) | rotated q part (rot)] per head, so a score is one
// dot product of rank + rot numbers and the attention's value is the row's first `rank` numbers.
//
// hb_latent_prepare: per token, the rotation of each head's rotated query part into the folded queries, and (for a
// layer that fills its cache entry) RMSNorm of the latent, rotation of the shared key part, and the write of both into
// the token's cache row. hb_latent_attention_generic: one warp per (query token, head) on CUDA cores, the float32
// engine's attention and the bfloat16 engine's for sizes its tensor-core kernel refuses.
#include "common.cuh"

template <typename T, typename TW>
__global__ void latent_prepare_kernel(T* __restrict__ qa, const T* __restrict__ first, int ld, int heads, int dim,
                                      int rot, int rank, int dkv_at, const int32_t* __restrict__ positions,
                                      const float* __restrict__ table, int rot_dims, int max_positions,
                                      const TW* __restrict__ norm_weight, float eps, T* __restrict__ cache,
                                      const int32_t* __restrict__ write_index, long cache_rows) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const T* fr = first + (size_t)t * ld;
    const int p = positions[t];
    const int half = rot_dims >> 1;
    const bool turn = half > 0 && p >= 0 && p < max_positions;
    const float* cs = table + (size_t)(turn ? p : 0) * rot_dims;           // cosines, then sines
    const int dk = rank + rot;
    if ((int)blockIdx.y < heads) {                     // this head's rotated query part -> qa[t, h, rank:]
        const int h = blockIdx.y;
        const T* q = fr + (size_t)h * (dim + rot) + dim;
        for (int d = threadIdx.x; d < rot; d += blockDim.x) {
            float v = to_f32(q[d]);
            if (turn && d < rot_dims) {
                const int j = d < half ? d : d - half;
                const float c = cs[j], s = cs[half + j];
                v = d < half ? v * c - to_f32(q[d + half]) * s : v * c + to_f32(q[d - half]) * s;
            }
            qa[((size_t)t * heads + h) * dk + rank + d] = from_f32<T>(v);
        }
        return;
    }
    if (dkv_at < 0) return;
    const long w = write_index[t];
    const T* d = fr + dkv_at;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(d[i]); ss += v * v; }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
    if (w < 0 || w >= cache_rows) return;
    T* row = cache + (size_t)w * dk;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_f32<T>(to_f32(d[i]) * rstd * to_f32(norm_weight[i]));
    const T* kr = d + rank;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float v = to_f32(kr[i]);
        if (turn && i < rot_dims) {
            const int j = i < half ? i : i - half;
            const float c = cs[j], s = cs[half + j];
            v = i < half ? v * c - to_f32(kr[i + half]) * s : v * c + to_f32(kr[i - half]) * s;
        }
        row[rank + i] = from_f32<T>(v);
    }
}

extern "C" int hb_latent_prepare(void* qa, const void* first, int dtype, int ld, int tokens, int heads, int dim, int rot,
                                 int rank, int dkv_at, const int32_t* positions, const float* table, int rot_dims,
                                 int max_positions, const void* norm_weight, int weight_dtype, float eps, void* cache,
                                 const int32_t* write_index, int pages, int page_size, hb_stream stream) {
    if (tokens == 0) return 0;
    if (rot_dims % 2 || rot_dims > rot || rot_dims < 0) HB_REFUSE("latent_prepare: %d of %d dimensions turn", rot_dims, rot);
    if (rot_dims && !table) HB_REFUSE("latent_prepare: a rotation needs its table");
    if (dkv_at >= 0 && (!cache || !write_index || !norm_weight)) HB_REFUSE("latent_prepare: a layer that fills its cache needs cache, write_index and the latent's norm weight");
    if (dkv_at >= 0 && dkv_at + rank + rot > ld) HB_REFUSE("latent_prepare: the down-projection's columns end past the row");
    cudaStream_t s = (cudaStream_t)stream;
    const long cache_rows = (long)pages * page_size;
    if (heads + 1 > 65535) HB_REFUSE("latent_prepare: %d heads", heads);
    dim3 grid(tokens, heads + (dkv_at >= 0 ? 1 : 0));      // a block a head, and one for the token's cache row
#define LP_GO(T_, TW_) latent_prepare_kernel<T_, TW_><<<grid, 128, 0, s>>>((T_*)qa, (const T_*)first, ld, heads, dim, rot, \
        rank, dkv_at, positions, table, rot_dims, max_positions, (const TW_*)norm_weight, eps, (T_*)cache, write_index, cache_rows)
    if (dtype == HB_F32) LP_GO(float, float);
    else if (dtype == HB_BF16 && weight_dtype == HB_F32) LP_GO(bf16, float);
    else if (dtype == HB_BF16) LP_GO(bf16, bf16);
    else HB_REFUSE("latent_prepare: dtype %d", dtype);
#undef LP_GO
    HB_LAUNCH_CHECK("latent_prepare");
    return 0;
}

// ---------------------------------------------------------------- attention on CUDA cores
#define LAT_WARPS 4
#define LAT_MAX_PER_LANE 32          // rank up to 1024

template <typename T>
__global__ void latent_attention_generic_kernel(T* __restrict__ out, const T* __restrict__ qa, const T* __restrict__ cache,
                                                const int32_t* __restrict__ block_table, int table_stride,
                                                const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
                                                const int32_t* __restrict__ kv_len, int rows, int tokens, int heads,
                                                int rank, int dk, int pages, int page_size, float scale, int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * LAT_WARPS + warp;
    if (item >= (long)tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    float* qs = smem + (size_t)warp * dk;

    int lo = 0, hi = rows;                           // the row b with query_start[b] <= t < query_start[b + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (query_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int n = kv_len[b];
    T* o = out + ((size_t)t * heads + h) * rank;
    const int pos = n - query_start[b + 1] + t;       // the query's position in its sequence
    if (n <= 0 || pos < 0) {
        for (int d = lane; d < rank; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const T* qr = qa + ((size_t)t * heads + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32(qr[d]) * scale;
    __syncwarp();

    const int32_t* table = block_table + (size_t)row_slot[b] * table_stride;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.f, acc[LAT_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < LAT_MAX_PER_LANE; ++i) acc[i] = 0.f;

    for (int j0 = first; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        long base = -1;                              // element offset of token j's cache row
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page >= 0 && page < pages) base = ((long)page * page_size + j % page_size) * dk;
        }
        float s = -INFINITY;
        if (base >= 0) {
            const T* kr = cache + base;
            float dot = 0.f;
            for (int d = 0; d < dk; ++d) dot += qs[d] * to_f32(kr[d]);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = m_new == -INFINITY ? 1.f : expf(m - m_new);
        const float p = base >= 0 ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < LAT_MAX_PER_LANE; ++i) acc[i] *= corr;
        const int count = min(32, pos - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long bj = __shfl_sync(0xffffffffu, base, jj);
            if (bj < 0) continue;
            const T* vr = cache + bj;                 // the value is the latent itself
#pragma unroll
            for (int i = 0; i < LAT_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] += pj * to_f32(vr[d]);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < LAT_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) o[d] = from_f32<T>(acc[i] * inv);
    }
}

extern "C" int hb_latent_attention_generic(void* out, const void* qa, const void* cache, int dtype,
                                           const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                           const int32_t* query_start, const int32_t* kv_len, int rows, int tokens,
                                           int heads, int rank, int rot, int pages, int page_size, float scale,
                                           int window, hb_stream stream) {
    if (tokens == 0 || rows == 0) return 0;
    if (rank > 32 * LAT_MAX_PER_LANE) HB_REFUSE("latent attention: rank %d is above %d", rank, 32 * LAT_MAX_PER_LANE);
    cudaStream_t s = (cudaStream_t)stream;
    const int dk = rank + rot;
    const long items = (long)tokens * heads;
    const unsigned blocks = (unsigned)((items + LAT_WARPS - 1) / LAT_WARPS);
    const size_t smem = (size_t)LAT_WARPS * dk * sizeof(float);
    if (dtype == HB_F32)
        latent_attention_generic_kernel<float><<<blocks, LAT_WARPS * 32, smem, s>>>(
            (float*)out, (const float*)qa, (const float*)cache, block_table, table_stride, row_slot, query_start, kv_len,
            rows, tokens, heads, rank, dk, pages, page_size, scale, window);
    else if (dtype == HB_BF16)
        latent_attention_generic_kernel<bf16><<<blocks, LAT_WARPS * 32, smem, s>>>(
            (bf16*)out, (const bf16*)qa, (const bf16*)cache, block_table, table_stride, row_slot, query_start, kv_len,
            rows, tokens, heads, rank, dk, pages, page_size, scale, window);
    else HB_REFUSE("latent attention: dtype %d", dtype);
    HB_LAUNCH_CHECK("latent_attention_generic");
    return 0;
}
