// Routed experts: the router's choice, the layout of (token, choice) pairs expert by expert, the experts' products
// over those rows, and the weighted sum back per token. Nothing is decided on the host: the number of rows an expert
// gets is only known on the device, so the products launch the most tiles the step can need and a tile that finds no
// rows returns at once.
//
// hb_route_top       z [tokens, ld] (32-bit logits) -> chosen [tokens, top], weight [tokens, top], counts[e] += 1
// hb_expert_rows     counts -> first row of every expert; place[pair] = its row, token_of[row] = its token
// hb_expert_linear   out[row] = act(x[token_of ? token_of[row] : row] · w[e(row)]ᵀ), any dtype, CUDA cores
// hb_expert_combine  out[t] = sum_k weight[t, k] · y[place[t, k]] (+ sigmoid(gate_t) · shared[t])
#include "common.cuh"

// ---------------------------------------------------------------- the router's choice
// One block per token. softmax over all experts in 32-bit; the `top` largest scores, equal scores by ascending
// expert; weight = score · scale, with `renormalize` divided by the chosen scores' sum first.
__global__ void route_top_kernel(int32_t* __restrict__ chosen, float* __restrict__ weight, int32_t* __restrict__ counts,
                                 const float* __restrict__ z, int ld, int experts, int top, float scale, int renormalize) {
    extern __shared__ float sc[];                       // experts scores
    __shared__ float scratch[33];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float* zr = z + (size_t)t * ld;
    float m = -INFINITY;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) m = fmaxf(m, zr[e]);
    m = block_max(m, scratch);
    float sum = 0.f;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { const float p = expf(zr[e] - m); sc[e] = p; sum += p; }
    sum = block_sum(sum, scratch);
    const float inv = 1.f / sum;
    float taken = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -1.f; int bi = 0x7fffffff;
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            const float v = sc[e];
            if (v > bv) { bv = v; bi = e; }              // (ascending e: the first of equals stays)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < warps; ++w)
                if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
            chosen[(size_t)t * top + k] = bi;
            weight[(size_t)t * top + k] = bv * inv;
            sc[bi] = -2.f;                               // out of the running
            atomicAdd(counts + bi, 1);
            taken += bv * inv;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float f = renormalize ? scale / taken : scale;
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= f;
    }
}

extern "C" int hb_route_top(int32_t* chosen, float* weight, int32_t* counts, const float* z, int ld, int tokens,
                            int experts, int top, float scale, int renormalize, hb_stream stream) {
    if (tokens == 0) return 0;
    if (experts < 1 || top < 1 || top > experts || ld < experts) HB_REFUSE("route_top: top %d of %d experts in rows of %d", top, experts, ld);
    if (experts > 8192) HB_REFUSE("route_top: %d experts are above 8192", experts);
    const int threads = experts > 256 ? 256 : experts > 64 ? 128 : 64;
    route_top_kernel<<<tokens, threads, (size_t)experts * sizeof(float), (cudaStream_t)stream>>>(
        chosen, weight, counts, z, ld, experts, top, scale, renormalize);
    HB_LAUNCH_CHECK("route_top");
    return 0;
}

// ---------------------------------------------------------------- rows expert by expert
// counts [2 experts + 1]: [0, experts) the tokens of each expert (from hb_route_top), [experts, 2 experts] receives the
// first row of each expert and the end. The counts are used as cursors meanwhile and hold the counts again afterwards.
__global__ void expert_starts_kernel(int32_t* counts, int experts) {
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int e0 = 0; e0 < experts; e0 += blockDim.x) {          // a block-wide scan, a stretch of blockDim.x at a time
        const int e = e0 + threadIdx.x;
        const int c = e < experts ? counts[e] : 0;
        int v = c;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        __shared__ int sums[32];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        if (lane == 31) sums[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int w = lane < (int)(blockDim.x >> 5) ? sums[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += u; }
            sums[lane] = w;
        }
        __syncthreads();
        const int before = carry + (warp ? sums[warp - 1] : 0) + v - c;
        if (e < experts) { counts[experts + e] = before; counts[e] = 0; }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + c;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[2 * experts] = carry;
}

__global__ void expert_scatter_kernel(int32_t* __restrict__ place, int32_t* __restrict__ token_of, int32_t* counts,
                                      const int32_t* __restrict__ chosen, int pairs, int top, int experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int e = chosen[i];
    if (e < 0 || e >= experts) { place[i] = -1; return; }
    const int p = counts[experts + e] + atomicAdd(counts + e, 1);
    place[i] = p;
    token_of[p] = i / top;
}

extern "C" int hb_expert_rows(int32_t* place, int32_t* token_of, int32_t* counts, const int32_t* chosen, int tokens,
                              int top, int experts, hb_stream stream) {
    if (tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    expert_starts_kernel<<<1, 256, 0, s>>>(counts, experts);
    HB_LAUNCH_CHECK("expert_starts");
    const int pairs = tokens * top;
    expert_scatter_kernel<<<(pairs + 255) / 256, 256, 0, s>>>(place, token_of, counts, chosen, pairs, top, experts);
    HB_LAUNCH_CHECK("expert_scatter");
    return 0;
}

// ---------------------------------------------------------------- the experts' products, any dtype, CUDA cores
__device__ __forceinline__ float expert_act(float v, int act) {
    if (act == 1) { v = fmaxf(v, 0.f); return v * v; }            // the square of relu
    if (act == 2) return v / (1.f + expf(-v));                   // silu
    return v;
}

#define EBM 64
#define EBN 64
#define EBK 16

// Finds the expert and the first row of m-tile `tile` (tiles of EBM rows, counted expert by expert); false: no such tile.
__device__ __forceinline__ bool expert_tile(const int32_t* __restrict__ starts, int experts, int tile, int bm, int& e_out,
                                            int& row0, int& row_end) {
    for (int e = 0; e < experts; ++e) {
        const int a = starts[e], b = starts[e + 1];
        const int tiles = (b - a + bm - 1) / bm;
        if (tile < tiles) { e_out = e; row0 = a + tile * bm; row_end = b; return true; }
        tile -= tiles;
    }
    return false;
}

template <typename T>
__global__ void __launch_bounds__(256) expert_linear_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                            const int32_t* __restrict__ token_of, const T* __restrict__ w,
                                                            const int32_t* __restrict__ starts, int experts, int n, int k,
                                                            int act) {
    __shared__ float xs[EBK][EBM + 4];
    __shared__ float ws[EBK][EBN + 4];
    __shared__ int src[EBM];
    __shared__ int tile_info[3];
    if (threadIdx.x == 0) {
        int e = 0, r0 = 0, r1 = 0;
        const bool ok = expert_tile(starts, experts, blockIdx.y, EBM, e, r0, r1);
        tile_info[0] = ok ? e : -1; tile_info[1] = r0; tile_info[2] = r1;
    }
    __syncthreads();
    const int e = tile_info[0], m0 = tile_info[1], m_end = tile_info[2];
    if (e < 0) return;
    const int tid = threadIdx.x;
    if (tid < EBM) src[tid] = m0 + tid < m_end ? (token_of ? token_of[m0 + tid] : m0 + tid) : -1;
    __syncthreads();
    const int n0 = blockIdx.x * EBN;
    const T* we = w + (size_t)e * n * k;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4] = {};
    const int xr = src[lr], wr = n0 + lr;
    for (int k0 = 0; k0 < k; k0 += EBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = k0 + lk + i;
            xs[lk + i][lr] = xr >= 0 && kk < k ? to_f32(x[(size_t)xr * k + kk]) : 0.f;
            ws[lk + i][lr] = wr < n && kk < k ? to_f32(we[(size_t)wr * k + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk2 = 0; kk2 < EBK; ++kk2) {
            const float4 a = *(const float4*)&xs[kk2][ty * 4];
            const float4 b = *(const float4*)&ws[kk2][tx * 4];
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= m_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < n) out[(size_t)r * n + c] = from_f32<T>(expert_act(acc[i][j], act));
        }
    }
}

extern "C" int hb_expert_linear(void* out, const void* x, int dtype, const int32_t* token_of, const void* w,
                                const int32_t* starts, int rows, int experts, int n, int k, int act, hb_stream stream) {
    if (rows == 0 || n == 0) return 0;
    if (k <= 0 || experts < 1) HB_REFUSE("expert_linear: k = %d, %d experts", k, experts);
    const long tiles = (rows + EBM - 1) / EBM + experts;          // the most m-tiles any split of the rows can have
    if (tiles > 65535) HB_REFUSE("expert_linear: %d rows over %d experts are above the kernel's limit", rows, experts);
    dim3 grid((n + EBN - 1) / EBN, (unsigned)tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32)
        expert_linear_kernel<float><<<grid, 256, 0, s>>>((float*)out, (const float*)x, token_of, (const float*)w, starts,
                                                          experts, n, k, act);
    else if (dtype == HB_BF16)
        expert_linear_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)out, (const bf16*)x, token_of, (const bf16*)w, starts,
                                                         experts, n, k, act);
    else HB_REFUSE("expert_linear: dtype %d", dtype);
    HB_LAUNCH_CHECK("expert_linear");
    return 0;
}

// ---------------------------------------------------------------- elementwise
template <typename T>
__global__ void activation_kernel(T* __restrict__ x, long count, int act) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = from_f32<T>(expert_act(to_f32(x[i]), act));
}

extern "C" int hb_activation(void* x, int dtype, long count, int act, hb_stream stream) {
    if (count == 0) return 0;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == HB_F32) activation_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float*)x, count, act);
    else if (dtype == HB_BF16) activation_kernel<bf16><<<blocks, 256, 0, (cudaStream_t)stream>>>((bf16*)x, count, act);
    else HB_REFUSE("activation: dtype %d", dtype);
    HB_LAUNCH_CHECK("activation");
    return 0;
}

// o[t, i] *= sigmoid(g[t * ld + i]) in 32-bit, rounded once.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, const T* __restrict__ g, int n, long ld) {
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) o[t * n + i] = from_f32<T>(to_f32(o[t * n + i]) / (1.f + expf(-to_f32(g[t * ld + i]))));
}

extern "C" int hb_sigmoid_gate(void* o, const void* g, int dtype, int tokens, int n, long ld, hb_stream stream) {
    if (tokens == 0 || n == 0) return 0;
    if (tokens > 65535) HB_REFUSE("sigmoid_gate: %d rows are above 65535", tokens);
    dim3 grid((n + 255) / 256, tokens);
    if (dtype == HB_F32) sigmoid_gate_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float*)o, (const float*)g, n, ld);
    else if (dtype == HB_BF16) sigmoid_gate_kernel<bf16><<<grid, 256, 0, (cudaStream_t)stream>>>((bf16*)o, (const bf16*)g, n, ld);
    else HB_REFUSE("sigmoid_gate: dtype %d", dtype);
    HB_LAUNCH_CHECK("sigmoid_gate");
    return 0;
}

// ---------------------------------------------------------------- the weighted sum per token
template <typename T>
__global__ void expert_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const int32_t* __restrict__ place,
                                      const float* __restrict__ weight, const T* __restrict__ shared,
                                      const float* __restrict__ z, int ldz, int gate_at, int top, int hidden) {
    const size_t t = blockIdx.x;
    const float gate = shared ? 1.f / (1.f + expf(-z[t * ldz + gate_at])) : 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = place[t * top + k];
            if (p >= 0) acc = fmaf(weight[t * top + k], to_f32(y[(size_t)p * hidden + i]), acc);
        }
        if (shared) acc = fmaf(gate, to_f32(shared[t * hidden + i]), acc);
        out[t * hidden + i] = from_f32<T>(acc);
    }
}

extern "C" int hb_expert_combine(void* out, const void* y, int dtype, const int32_t* place, const float* weight,
                                 const void* shared, const float* z, int ldz, int gate_at, int tokens, int top, int hidden,
                                 hb_stream stream) {
    if (tokens == 0) return 0;
    if (shared && (!z || gate_at >= ldz)) HB_REFUSE("expert_combine: a shared expert needs its gate's logit");
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32)
        expert_combine_kernel<float><<<tokens, threads, 0, s>>>((float*)out, (const float*)y, place, weight,
                                                                (const float*)shared, z, ldz, gate_at, top, hidden);
    else if (dtype == HB_BF16)
        expert_combine_kernel<bf16><<<tokens, threads, 0, s>>>((bf16*)out, (const bf16*)y, place, weight,
                                                               (const bf16*)shared, z, ldz, gate_at, top, hidden);
    else HB_REFUSE("expert_combine: dtype %d", dtype);
    HB_LAUNCH_CHECK("expert_combine");
    return 0;
}
