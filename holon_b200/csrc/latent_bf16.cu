// Latent attention in bfloat16 on tensor cores (mma.sync m16n8k16, 32-bit scores, softmax and sums), for rows that
// bring any number of tokens: prompt portions and single decoded tokens.
//
// All heads read the same cache rows [latent (rank) | rotated key part (rot)], so a request's (token, head) pairs are
// the M side of one problem: its folded queries qa [tokens, heads, rank + rot] are contiguous rows of rank + rot, a
// tile of them meets a tile of 64 cache rows once for the scores (over rank + rot) and once more, the same rows in
// shared memory, for the values (their first `rank` numbers). A CTA has W = 4 warps (rows of one token: few query
// rows, many CTAs) or 8 (prompt portions: a larger tile reads the cache rows once for twice the queries). The output's
// `rank` columns are cut into R = 1, 2 or 4 parts of up to 128; a warp owns 16 query rows and one part, so a CTA's
// tile is 16 W / R rows, the R warps of a row group hold the same scores and run the same softmax
// and each adds up its own columns. (The scores themselves are shared out: each of the R warps multiplies the queries
// with 64 / R of the tile's cache rows, and the group exchanges the results through shared memory.) Cache rows arrive by cp.async, two tiles in flight; rows past a request's length are zero-filled.
// With `splits` > 1 (few query rows, many keys: decoding) a CTA takes one part of the key tiles and leaves its
// running maximum, sum and unnormalised output in scratch; a second kernel merges the parts in a fixed order.
#include "common.cuh"

#define LB_BN 64                       // cache rows a tile
#define LB_SLD 68                      // floats a row of exchanged scores

__device__ __forceinline__ void lb_cp16(void* dst, const void* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void lb_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lb_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void lb_ldsm4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lb_ldsm4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lb_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lb_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}

template <int R, int W>
__global__ void __launch_bounds__(W * 32, 1) latent_attention_bf16_kernel(
        bf16* __restrict__ out, float* __restrict__ scratch, const bf16* __restrict__ qa, const bf16* __restrict__ cache,
        const int32_t* __restrict__ block_table, int table_stride, const int32_t* __restrict__ row_slot,
        const int32_t* __restrict__ query_start, const int32_t* __restrict__ kv_len, int row0, int row1, int heads,
        int rank, int dk, int pages, int page_size, float scale, int window, int splits) {
    constexpr int MT = 16 * W / R;                         // query rows a CTA
    constexpr int LB_THREADS = W * 32;
    extern __shared__ __align__(16) unsigned char lb_smem[];
    __shared__ long kb[2][LB_BN];                          // element offset of each cache row of a stage (-1: none)
    const int ld = dk + 8;                                 // shared-memory row stride: 16 bytes of padding a row
    bf16* qs = (bf16*)lb_smem;                             // [MT][ld]
    bf16* ks = qs + (size_t)MT * ld;                       // [2][LB_BN][ld]
    float* sbuf = (float*)(ks + (size_t)2 * LB_BN * ld);   // [W / R][16][LB_SLD]: a row group's scores (R > 1)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // which request and which tile of its (token, head) pairs
    int tile = blockIdx.x, b = row0, nq = 0, n_flat = 0;
    for (; b < row1; ++b) {
        nq = query_start[b + 1] - query_start[b];
        n_flat = nq * heads;
        const int tiles = (n_flat + MT - 1) / MT;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (b >= row1) return;
    const int split = blockIdx.y;
    const int n = kv_len[b], q0 = query_start[b];
    const int flat0 = tile * MT;
    const long flat_global = (long)q0 * heads + flat0;      // the tile's first row among all (token, head) pairs
    const int rows_here = min(MT, n_flat - flat0);
    const int pos0 = n - nq;                                // position of the request's first new token
    const int t_first = flat0 / heads, t_last = (flat0 + rows_here - 1) / heads;
    const int key_hi = min(n, pos0 + t_last + 1);           // keys [key_lo, key_hi) are seen by some row of the tile
    const int key_lo = window > 0 ? max(0, pos0 + t_first - window + 1) : 0;
    const int tile_first = key_lo / LB_BN, tile_end = (key_hi + LB_BN - 1) / LB_BN;
    const int per = (max(0, tile_end - tile_first) + splits - 1) / splits;
    const int my_first = tile_first + split * per, my_end = min(tile_end, my_first + per);
    const int32_t* table = block_table + (size_t)row_slot[b] * table_stride;
    const int chunks = dk >> 3;                             // 16-byte pieces a row

    // the queries: MT contiguous rows of dk
    for (int c = tid; c < MT * chunks; c += LB_THREADS) {
        const int r = c / chunks, col = (c % chunks) * 8;
        const bool ok = r < rows_here;
        lb_cp16(qs + (size_t)r * ld + col, qa + (flat_global + (ok ? r : 0)) * dk + col, ok ? 16 : 0);
    }
    lb_commit();

    auto load_keys = [&](int kt, int stage) {
        if (tid < LB_BN) {
            const int j = kt * LB_BN + tid;
            long base = -1;
            if (j < n) {
                const int page = table[j / page_size];
                if (page >= 0 && page < pages) base = ((long)page * page_size + j % page_size) * dk;
            }
            kb[stage][tid] = base;
        }
        __syncthreads();
        bf16* dst = ks + (size_t)stage * LB_BN * ld;
        for (int c = tid; c < LB_BN * chunks; c += LB_THREADS) {
            const int r = c / chunks, col = (c % chunks) * 8;
            const long base = kb[stage][r];
            lb_cp16(dst + (size_t)r * ld + col, cache + (base >= 0 ? base + col : 0), base >= 0 ? 16 : 0);
        }
        lb_commit();
    };

    const int group = warp / R, part = warp % R;
    const int part_cols = ((rank / R + 15) / 16) * 16;      // columns a warp owns (the last part may own fewer)
    const int col0 = part * part_cols;
    const int pairs = max(0, min(part_cols, rank - col0)) / 16;     // 16-column pairs of this warp, up to 8
    const float sl2 = scale * 1.4426950408889634f;
    const int r_lo = group * 16 + (lane >> 2), r_hi = r_lo + 8;     // this thread's two query rows within the tile
    const int pos_lo = pos0 + (flat0 + r_lo) / heads, pos_hi = pos0 + (flat0 + r_hi) / heads;
    const bool live_lo = r_lo < rows_here, live_hi = r_hi < rows_here;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    if (my_first < my_end) load_keys(my_first, 0);
    for (int kt = my_first; kt < my_end; ++kt) {
        const int stage = (kt - my_first) & 1;
        if (kt + 1 < my_end) { load_keys(kt + 1, stage ^ 1); lb_wait<1>(); } else { lb_wait<0>(); }
        __syncthreads();
        const bf16* kt_s = ks + (size_t)stage * LB_BN * ld;
        // scores of this warp's 16 rows against the tile's 64 cache rows: each of the R warps of a row group takes
        // 64 / R of the cache rows and the group exchanges the scores through shared memory
        float s[8][4];
        {
            constexpr int NP = 4 / R;                       // 16-row pairs of cache rows this warp scores
            float sp[2 * NP][4];
#pragma unroll
            for (int i = 0; i < 2 * NP; ++i) { sp[i][0] = sp[i][1] = sp[i][2] = sp[i][3] = 0.f; }
            const int key0 = part * NP * 16;
            int kk = 0;
            if constexpr (NP <= 2) {
                // few cache rows a warp: two sets of sums over alternate steps of 16, so that a product does not wait
                // for the one before it (the sets are added below)
                float sq[2 * NP][4];
#pragma unroll
                for (int i = 0; i < 2 * NP; ++i) { sq[i][0] = sq[i][1] = sq[i][2] = sq[i][3] = 0.f; }
#pragma unroll 2
                for (; kk + 32 <= dk; kk += 32) {
                    uint32_t a0[4], a1[4];
                    lb_ldsm4(a0, qs + (size_t)(group * 16 + (lane & 15)) * ld + kk + (lane >> 4) * 8);
                    lb_ldsm4(a1, qs + (size_t)(group * 16 + (lane & 15)) * ld + kk + 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        uint32_t b0[4], b1[4];
                        const bf16* kr = kt_s + (size_t)(key0 + q * 16 + (lane & 7) + (lane >> 4) * 8) * ld + kk + ((lane >> 3) & 1) * 8;
                        lb_ldsm4(b0, kr);
                        lb_ldsm4(b1, kr + 16);
                        lb_mma(sp[2 * q], a0, b0[0], b0[1]);
                        lb_mma(sq[2 * q], a1, b1[0], b1[1]);
                        lb_mma(sp[2 * q + 1], a0, b0[2], b0[3]);
                        lb_mma(sq[2 * q + 1], a1, b1[2], b1[3]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 2 * NP; ++i) { sp[i][0] += sq[i][0]; sp[i][1] += sq[i][1]; sp[i][2] += sq[i][2]; sp[i][3] += sq[i][3]; }
            }
            for (; kk < dk; kk += 16) {
                uint32_t a[4];
                lb_ldsm4(a, qs + (size_t)(group * 16 + (lane & 15)) * ld + kk + (lane >> 4) * 8);
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    uint32_t bfr[4];
                    lb_ldsm4(bfr, kt_s + (size_t)(key0 + q * 16 + (lane & 7) + (lane >> 4) * 8) * ld + kk + ((lane >> 3) & 1) * 8);
                    lb_mma(sp[2 * q], a, bfr[0], bfr[1]);
                    lb_mma(sp[2 * q + 1], a, bfr[2], bfr[3]);
                }
            }
            if constexpr (R == 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { s[i][0] = sp[i][0]; s[i][1] = sp[i][1]; s[i][2] = sp[i][2]; s[i][3] = sp[i][3]; }
            } else {
                float* sg = sbuf + (size_t)group * 16 * LB_SLD;
#pragma unroll
                for (int i = 0; i < 2 * NP; ++i) {
                    const int col = key0 + i * 8 + (lane & 3) * 2;
                    *(float2*)(sg + (size_t)(lane >> 2) * LB_SLD + col) = make_float2(sp[i][0], sp[i][1]);
                    *(float2*)(sg + (size_t)((lane >> 2) + 8) * LB_SLD + col) = make_float2(sp[i][2], sp[i][3]);
                }
                asm volatile("bar.sync %0, %1;\n" ::"r"(1 + group), "r"(R * 32));      // the R warps of this row group
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 lo = *(const float2*)(sg + (size_t)(lane >> 2) * LB_SLD + i * 8 + (lane & 3) * 2);
                    const float2 hi = *(const float2*)(sg + (size_t)((lane >> 2) + 8) * LB_SLD + i * 8 + (lane & 3) * 2);
                    s[i][0] = lo.x; s[i][1] = lo.y; s[i][2] = hi.x; s[i][3] = hi.y;
                }
            }
        }
        // mask, running maximum and sum (two rows a thread, four threads a row)
        const int j0 = kt * LB_BN + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + i * 8 + e;
                const bool see_lo = live_lo && j <= pos_lo && (window <= 0 || pos_lo - j < window);
                const bool see_hi = live_hi && j <= pos_hi && (window <= 0 || pos_hi - j < window);
                s[i][e] = see_lo ? s[i][e] * sl2 : -INFINITY;
                s[i][2 + e] = see_hi ? s[i][2 + e] * sl2 : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[i][e]);
                mx_hi = fmaxf(mx_hi, s[i][2 + e]);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float new_lo = fmaxf(m_lo, mx_lo), new_hi = fmaxf(m_hi, mx_hi);
        const float ref_lo = new_lo == -INFINITY ? 0.f : new_lo, ref_hi = new_hi == -INFINITY ? 0.f : new_hi;
        const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);      // (m = -inf at the start: 0)
        m_lo = new_lo; m_hi = new_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[i][e] = exp2f(s[i][e] - ref_lo);
                s[i][2 + e] = exp2f(s[i][2 + e] - ref_hi);
                sum_lo += s[i][e];
                sum_hi += s[i][2 + e];
            }
        }
        l_lo = l_lo * c_lo + sum_lo;                        // (each thread keeps its own quarter of the row's sum)
        l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < 16; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
        // the values: the same cache rows, columns col0 .. of the latent
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
            uint32_t a[4];
            a[0] = lb_pack(s[2 * k2][0], s[2 * k2][1]);
            a[1] = lb_pack(s[2 * k2][2], s[2 * k2][3]);
            a[2] = lb_pack(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
            a[3] = lb_pack(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                if (p < pairs) {
                    uint32_t bfr[4];
                    lb_ldsm4_t(bfr, kt_s + (size_t)(k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + col0 + p * 16 + (lane >> 4) * 8);
                    lb_mma(o[2 * p], a, bfr[0], bfr[1]);
                    lb_mma(o[2 * p + 1], a, bfr[2], bfr[3]);
                }
            }
        }
        __syncthreads();                                    // the stage is free for the load after next
    }
    lb_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    const int cq = (lane & 3) * 2;
    if (splits == 1) {
        const float i_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            if (p < 2 * pairs) {
                const int col = col0 + p * 8 + cq;
                if (live_lo) *(__nv_bfloat162*)(out + (flat_global + r_lo) * rank + col) = __floats2bfloat162_rn(o[p][0] * i_lo, o[p][1] * i_lo);
                if (live_hi) *(__nv_bfloat162*)(out + (flat_global + r_hi) * rank + col) = __floats2bfloat162_rn(o[p][2] * i_hi, o[p][3] * i_hi);
            }
        }
        return;
    }
    // partial results: [pair row][split][m, l, rank columns], base-2 maximum
    const int width = rank + 2;
    float* p_lo = scratch + ((flat_global + r_lo) * splits + split) * width;
    float* p_hi = scratch + ((flat_global + r_hi) * splits + split) * width;
    if (part == 0 && (lane & 3) == 0) {
        if (live_lo) { p_lo[0] = m_lo; p_lo[1] = l_lo; }
        if (live_hi) { p_hi[0] = m_hi; p_hi[1] = l_hi; }
    }
#pragma unroll
    for (int p = 0; p < 16; ++p) {
        if (p < 2 * pairs) {
            const int col = 2 + col0 + p * 8 + cq;
            if (live_lo) { p_lo[col] = o[p][0]; p_lo[col + 1] = o[p][1]; }
            if (live_hi) { p_hi[col] = o[p][2]; p_hi[col + 1] = o[p][3]; }
        }
    }
}

// One block per (token, head) pair: the parts' weights first (their maxima and sums, in the order of the parts), then
// every thread adds up its columns over the parts.
#define LB_MERGE_MAX 64
__global__ void __launch_bounds__(512) latent_attention_merge_kernel(bf16* __restrict__ out, const float* __restrict__ scratch,
                                                                     long first_pair, int rank, int splits) {
    __shared__ float wgt[LB_MERGE_MAX];
    __shared__ float inv_l;
    const long i = first_pair + blockIdx.x;
    const int width = rank + 2;
    const float* p = scratch + i * splits * width;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m = -INFINITY;
        for (int s = lane; s < splits; s += 32) m = fmaxf(m, p[(size_t)s * width]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = lane; s < splits; s += 32) {
            const float ms = p[(size_t)s * width];
            const float w = ms == -INFINITY ? 0.f : exp2f(ms - m);
            wgt[s] = w;
            l += w * p[(size_t)s * width + 1];
        }
        l = warp_sum(l);
        if (lane == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
    }
    __syncthreads();
    const float inv = inv_l;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) acc = fmaf(wgt[s], p[(size_t)s * width + 2 + c], acc);
        out[i * rank + c] = __float2bfloat16_rn(acc * inv);
    }
}

extern "C" size_t hb_latent_attention_scratch_floats(int tokens, int heads, int rank, int splits) {
    return splits > 1 ? (size_t)tokens * heads * splits * (rank + 2) : 0;
}

// Rows row0 .. row1 - 1 of the batch, which bring `tokens` tokens in all, the first of them token `first_token` of the
// step. rank and rot multiples of 16, rank up to 512. splits > 1: scratch of hb_latent_attention_scratch_floats(all
// tokens of the step, ...) floats.
extern "C" int hb_latent_attention_bf16(void* out, float* scratch, const void* qa, const void* cache,
                                        const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                        const int32_t* query_start, const int32_t* kv_len, int row0, int row1,
                                        int first_token, int tokens, int heads, int rank, int rot, int pages,
                                        int page_size, float scale, int window, int splits, hb_stream stream) {
    if (tokens == 0 || row1 <= row0) return 0;
    const int dk = rank + rot;
    if (rank % 16 || rot % 16 || rank < 16 || rank > 512) HB_REFUSE("latent attention on tensor cores: rank %d and rot %d must be multiples of 16, rank 16 to 512", rank, rot);
    if (((uintptr_t)qa | (uintptr_t)cache | (uintptr_t)out) % 16) HB_REFUSE("latent attention on tensor cores: pointers must be 16-byte aligned");
    if (splits < 1 || splits > LB_MERGE_MAX || (splits > 1 && !scratch)) HB_REFUSE("latent attention: %d splits (1 to %d; more than one need scratch)", splits, LB_MERGE_MAX);
    cudaStream_t s = (cudaStream_t)stream;
    const int r = rank <= 128 ? 1 : rank <= 256 ? 2 : 4;
    const int warps = tokens > row1 - row0 ? 8 : 4;                     // (rows of several tokens: the larger tile)
    const int mt = 16 * warps / r;
    const long pairs = (long)tokens * heads;
    const long tiles = (pairs + mt - 1) / mt + (row1 - row0);          // the most tiles any cut of the tokens into the rows has
    if (tiles > 0x7fffffffL || splits > 65535) HB_REFUSE("latent attention: %ld tiles, %d splits", tiles, splits);
    const size_t smem = (size_t)(mt + 2 * LB_BN) * (dk + 8) * sizeof(bf16) + (r > 1 ? (size_t)(warps / r) * 16 * LB_SLD * sizeof(float) : 0);
    dim3 grid((unsigned)tiles, (unsigned)splits);
#define LB_GO(R_, W_) do { \
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(latent_attention_bf16_kernel<R_, W_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        latent_attention_bf16_kernel<R_, W_><<<grid, W_ * 32, smem, s>>>((bf16*)out, scratch, (const bf16*)qa, (const bf16*)cache, \
            block_table, table_stride, row_slot, query_start, kv_len, row0, row1, heads, rank, dk, pages, page_size, scale, window, splits); \
    } while (0)
    if (warps == 4) { if (r == 1) LB_GO(1, 4); else if (r == 2) LB_GO(2, 4); else LB_GO(4, 4); }
    else { if (r == 1) LB_GO(1, 8); else if (r == 2) LB_GO(2, 8); else LB_GO(4, 8); }
#undef LB_GO
    HB_LAUNCH_CHECK("latent_attention_bf16");
    if (splits > 1) {
        latent_attention_merge_kernel<<<(unsigned)pairs, min(512, (rank + 31) / 32 * 32), 0, s>>>((bf16*)out, scratch, (long)first_token * heads, rank, splits);
        HB_LAUNCH_CHECK("latent_attention_merge");
    }
    return 0;
}
