// Hyper-connections: S copies of the residual per token, mixed by learned coefficients around every sublayer.
// One kernel does what the residual sum and the norm do for a single stream: it folds the pending sublayer output y
// into all streams at once (new_t = sum_s mix[s, t] old_s + out[t] y), writes them, reads them with the next
// sublayer's coefficients (u = sum_t in[t] new_t) and leaves RMSNorm(u) for the next product. All in 32-bit; the
// streams are 32-bit in memory. One block per row; u is kept in shared memory between the two passes.
#include "common.cuh"

#define HC_MAX_STREAMS 16

struct hc_coef {
    float mix[HC_MAX_STREAMS * HC_MAX_STREAMS];
    float out[HC_MAX_STREAMS];
    float in[HC_MAX_STREAMS];
};

template <typename TD, typename TW, int S>
__global__ void __launch_bounds__((S > 0 && S <= 4) ? 1024 : 256) hyper_mix_norm_kernel(TD* __restrict__ out, float* xs, const float* __restrict__ src,
                                      const TD* __restrict__ y, const float* __restrict__ mix,
                                      const float* __restrict__ outc, const float* __restrict__ inc,
                                      const TW* __restrict__ weight, float eps, float offset,
                                      const int32_t* __restrict__ index, int dim, int streams) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    __shared__ hc_coef c;
    const int n = S > 0 ? S : streams;
    const int r = blockIdx.x;
    const size_t t = index ? (size_t)index[r] : (size_t)r;
    const bool fold = y != nullptr, write = index == nullptr && (fold || src != nullptr);
    float* xr = xs + t * (size_t)n * dim;
    if constexpr (S > 0 && S <= 4) {
        if (dim <= (int)blockDim.x * 4) {
            // A row that the block's threads hold whole (four columns a thread): coefficients straight from global
            // memory, every load of the row in flight at once, the norm's weight read before the block-wide sum; the
            // values and their order are those of the general path below.
            float cm[S * S], co[S], ci[S];
#pragma unroll
            for (int i = 0; i < S * S; ++i) cm[i] = mix ? __ldg(mix + i) : 0.f;
#pragma unroll
            for (int i = 0; i < S; ++i) { co[i] = outc ? __ldg(outc + i) : 0.f; ci[i] = inc ? __ldg(inc + i) : 1.f; }
            float old[4][S], yv[4], wv[4], u[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                if (i < dim) {
#pragma unroll
                    for (int q = 0; q < S; ++q) old[k][q] = src ? src[t * dim + i] : xr[(size_t)q * dim + i];
                    yv[k] = fold ? to_f32(y[t * dim + i]) : 0.f;
                    wv[k] = to_f32(weight[i]) + offset;
                }
            }
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                u[k] = 0.f;
                if (i < dim) {
#pragma unroll
                    for (int q = 0; q < S; ++q) {
                        float v;
                        if (fold) {
                            v = 0.f;
#pragma unroll
                            for (int p = 0; p < S; ++p) v = fmaf(cm[p * S + q], old[k][p], v);
                            v = fmaf(co[q], yv[k], v);
                        } else {
                            v = old[k][q];
                        }
                        if (write) xr[(size_t)q * dim + i] = v;
                        u[k] = fmaf(ci[q], v, u[k]);
                    }
                    ss += u[k] * u[k];
                }
            }
            const float rstd = rsqrtf(block_sum(ss, scratch) / (float)dim + eps);
            TD* o = out + (size_t)r * dim;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                if (i < dim) o[i] = from_f32<TD>(u[k] * rstd * wv[k]);
            }
            return;
        }
    }
    for (int i = threadIdx.x; i < n * n; i += blockDim.x) c.mix[i] = mix ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        c.out[i] = outc ? outc[i] : 0.f;
        c.in[i] = inc ? inc[i] : 1.f;
    }
    __syncthreads();
    float ss = 0.f;
    constexpr int NS = S > 0 ? S : HC_MAX_STREAMS;
    constexpr int U = S > 0 && S <= 4 ? 4 : 1;              // columns a thread has in flight at once
    for (int i0 = threadIdx.x; i0 < dim; i0 += blockDim.x * U) {
        float old[U][NS], yv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {                       // every load of this pass first
            const int i = i0 + u * blockDim.x;
            if (i < dim) {
                if (src) {
                    const float v = src[t * dim + i];
#pragma unroll
                    for (int s = 0; s < NS; ++s) if (s < n) old[u][s] = v;
                } else {
#pragma unroll
                    for (int s = 0; s < NS; ++s) if (s < n) old[u][s] = xr[(size_t)s * dim + i];
                }
                yv[u] = fold ? to_f32(y[t * dim + i]) : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i >= dim) continue;
            float acc = 0.f;
#pragma unroll
            for (int q = 0; q < NS; ++q) {
                if (q >= n) break;
                float v;
                if (fold) {
                    v = 0.f;
#pragma unroll
                    for (int s = 0; s < NS; ++s) if (s < n) v = fmaf(c.mix[s * n + q], old[u][s], v);
                    v = fmaf(c.out[q], yv[u], v);
                } else {
                    v = old[u][q];
                }
                if (write) xr[(size_t)q * dim + i] = v;
                acc = fmaf(c.in[q], v, acc);
            }
            row[i] = acc;
            ss += acc * acc;
        }
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)dim + eps);
    TD* o = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TD>(row[i] * rstd * (to_f32(weight[i]) + offset));
}

template <typename TD, typename TW>
static int hyper_launch(void* out, float* xs, const float* src, const void* y, const float* mix, const float* outc,
                        const float* inc, const void* weight, float eps, float offset, const int32_t* index, int rows,
                        int dim, int streams, cudaStream_t s) {
    // up to four streams: four columns a thread hold a whole row of up to 4,096; more streams: the kernel with many registers
    const int wide = dim > 2048 && rows <= 512 ? 1024 : dim > 1024 ? 512 : dim > 512 ? 256 : 128;   // (many rows: blocks of 512 fill the SMs better)
    const int threads = streams <= 4 ? wide : (wide < 256 ? wide : 256);
    const size_t smem = (size_t)dim * sizeof(float);
#define HC_GO(S_) hyper_mix_norm_kernel<TD, TW, S_><<<rows, threads, smem, s>>>((TD*)out, xs, src, (const TD*)y, mix, outc, \
        inc, (const TW*)weight, eps, offset, index, dim, streams)
#define HC_CASE(S_) case S_: \
        if (smem > 48 * 1024 && cudaFuncSetAttribute(hyper_mix_norm_kernel<TD, TW, S_ % HC_MAX_STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            HB_REFUSE("hyper_mix_norm: %d columns do not fit in shared memory", dim); \
        HC_GO(S_ % HC_MAX_STREAMS); break
    switch (streams <= 4 || streams == 8 ? streams : HC_MAX_STREAMS) {      // (16 stands for the kernel of any number)
        HC_CASE(1); HC_CASE(2); HC_CASE(3); HC_CASE(4); HC_CASE(8);
        default: HC_CASE(16);
    }
#undef HC_CASE
#undef HC_GO
    HB_LAUNCH_CHECK("hyper_mix_norm");
    return 0;
}

// Row r reads token t = index ? index[r] : r. Old streams: xs [tokens, streams, dim], or, with src [tokens, dim], that
// row for every stream. With y [tokens, dim] (out's dtype): new_q = sum_s mix[s * streams + q] old_s + outc[q] y, else
// new = old. Without index the new streams are written to xs. out [rows, dim] = RMSNorm(sum_q inc[q] new_q) (inc null:
// ones) times (weight + offset).
extern "C" int hb_hyper_mix_norm(void* out, int out_dtype, float* xs, const float* src, const void* y, const float* mix,
                                 const float* outc, const float* inc, const void* weight, int weight_dtype, float eps,
                                 float offset, const int32_t* index, int rows, int dim, int streams, hb_stream stream) {
    if (rows == 0) return 0;
    if (streams < 1 || streams > HC_MAX_STREAMS) HB_REFUSE("hyper_mix_norm: %d streams; 1 to %d", streams, HC_MAX_STREAMS);
    if (y && (!mix || !outc)) HB_REFUSE("hyper_mix_norm: a pending output needs its mix and out coefficients");
    if (dim > 51200) HB_REFUSE("hyper_mix_norm: %d columns are above 51200", dim);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_F32 && weight_dtype == HB_F32)
        return hyper_launch<float, float>(out, xs, src, y, mix, outc, inc, weight, eps, offset, index, rows, dim, streams, s);
    if (out_dtype == HB_BF16 && weight_dtype == HB_BF16)
        return hyper_launch<bf16, bf16>(out, xs, src, y, mix, outc, inc, weight, eps, offset, index, rows, dim, streams, s);
    if (out_dtype == HB_BF16 && weight_dtype == HB_F32)
        return hyper_launch<bf16, float>(out, xs, src, y, mix, outc, inc, weight, eps, offset, index, rows, dim, streams, s);
    HB_REFUSE("hyper_mix_norm: out dtype %d with weight dtype %d", out_dtype, weight_dtype);
}
