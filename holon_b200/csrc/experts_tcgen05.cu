// The experts' products for prompts on tcgen05 tensor cores: csrc/gemm_tcgen05.cu's kernel (TMA into a four-stage
// ring, one thread issuing 128 x 256 x 16 MMAs into two alternating tensor-memory accumulators, four epilogue warps)
// over tiles that are counted expert by expert. The rows of all experts lie one after the other (x is gathered into
// that order first, where it is not in it already), so a tile's 128 rows of x are one TMA box starting at the
// expert's m-th block of rows, and its 256 weight rows one pair of boxes in the stacked weight [experts * n, k]
// starting at e * n. A box may run past its expert's last row (into the next expert's rows or weights, or past the
// end, where TMA fills zeros): those rows and columns are computed and not stored. Which tiles there are is only known
// on the device: a small kernel lists them (expert, first row, the expert's end), the product launches persistent
// CTAs over the most tiles any split of the rows can have, and every role stops at the first tile the list leaves empty.
// Every wait is bounded as in the other tcgen05 kernels (status word: hb_experts_tcgen05_status).
#include "tcgen05.cuh"

#define XT_BM 128
#define XT_BN 256
#define XT_BK 64
#define XT_STAGES 4
#define XT_A_BYTES (XT_BM * XT_BK * 2)
#define XT_B_BYTES (XT_BN * XT_BK * 2)
#define XT_STAGE_BYTES (XT_A_BYTES + XT_B_BYTES)
#define XT_SMEM (XT_STAGES * XT_STAGE_BYTES + 1024 + 256)

// table [max_tiles][3]: expert (-1: no such tile), first row, the expert's end. One warp.
__global__ void expert_tiles_kernel(int32_t* __restrict__ table, const int32_t* __restrict__ starts, int experts, int max_tiles) {
    const int lane = threadIdx.x;
    int base = 0;
    for (int e0 = 0; e0 < experts; e0 += 32) {
        const int e = e0 + lane;
        const int a = e < experts ? starts[e] : 0, b = e < experts ? starts[e + 1] : 0;
        const int tiles = (b - a + XT_BM - 1) / XT_BM;
        int incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
        const int before = base + incl - tiles;
        for (int i = 0; i < tiles; ++i) {
            const int at = before + i;
            if (at < max_tiles) { table[3 * at] = e; table[3 * at + 1] = a + i * XT_BM; table[3 * at + 2] = b; }
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
    for (int at = base + lane; at < max_tiles; at += 32) table[3 * at] = -1;
}

__global__ void gather_rows_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, const int32_t* __restrict__ token_of, int k) {
    const size_t r = blockIdx.x;
    const uint4* src = (const uint4*)(x + (size_t)token_of[r] * k);
    uint4* dst = (uint4*)(out + r * k);
    for (int c = threadIdx.x; c < (k >> 3); c += blockDim.x) dst[c] = __ldg(src + c);
}

__device__ __forceinline__ float xt_act(float v, int act) {
    if (act == 1) { v = fmaxf(v, 0.f); return v * v; }
    if (act == 2) return v / (1.f + __expf(-v));
    return v;
}

__global__ void __launch_bounds__(192, 1) expert_linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       bf16* __restrict__ out, const int32_t* __restrict__ table,
                                                                       int n, int k, int act, int tiles_m, int tiles_n) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + XT_STAGES * XT_STAGE_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * XT_STAGES;
    const uint32_t acc_full0 = bars + 16 * XT_STAGES, acc_empty0 = acc_full0 + 16;
    const uint32_t slot = acc_empty0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (k + XT_BK - 1) / XT_BK;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < XT_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(2 * XT_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));

    // tile t: m-tile t / tiles_n of the list (n-tiles of one block of rows run side by side and share it in the L2)
    if (warp == 0) {
        if (lane == 0) {
            int kb_all = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                const int mt = t / tiles_n, nt = t - mt * tiles_n;
                const int e = table[3 * mt];
                if (e < 0) break;                                     // (the list's tiles are its first entries)
                const int m0 = table[3 * mt + 1];
                const int w0 = e * n + nt * XT_BN, w1 = w0 + 128;
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb, ++kb_all) {
                    const int s = kb_all % XT_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((kb_all / XT_STAGES) & 1) ^ 1, 1);
                    if (!ok) break;
                    const uint32_t a = base + s * XT_STAGE_BYTES, b = a + XT_A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, XT_STAGE_BYTES);
                    tma_load_2d(a, &map_x, full0 + 8 * s, kb * XT_BK, m0);
                    tma_load_2d(b, &map_w, full0 + 8 * s, kb * XT_BK, w0);
                    tma_load_2d(b + XT_B_BYTES / 2, &map_w, full0 + 8 * s, kb * XT_BK, w1);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(XT_BN >> 3) << 17) | ((uint32_t)(XT_BM >> 4) << 24);
            int kb_all = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
                if (table[3 * (t / tiles_n)] < 0) break;
                const int acc = local & 1, use = local >> 1;
                ok = mbar_wait(acc_empty0 + 8 * acc, (use & 1) ^ 1, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * XT_BN;
                for (int kb = 0; kb < kblocks; ++kb, ++kb_all) {
                    const int s = kb_all % XT_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (kb_all / XT_STAGES) & 1, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a = base + s * XT_STAGE_BYTES, b = a + XT_A_BYTES;
                    const uint64_t da = tc_smem_desc(a), db = tc_smem_desc(b);
#pragma unroll
                    for (int kk = 0; kk < XT_BK / 16; ++kk)
                        tc_mma(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0);
                    tc_commit(empty0 + 8 * s);
                }
                tc_commit(acc_full0 + 8 * acc);
            }
        }
    } else {
        const int q = warp & 3;
        int local = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++local) {
            const int mt = t / tiles_n, nt = t - mt * tiles_n;
            if (table[3 * mt] < 0) break;
            const int acc = local & 1, use = local >> 1;
            const int row = table[3 * mt + 1] + q * 32 + lane, row_end = table[3 * mt + 2];
            const int col0 = nt * XT_BN;
            if (!mbar_wait(acc_full0 + 8 * acc, use & 1, 3)) break;
            tc_fence_after();
            const uint32_t d = tmem + acc * XT_BN + ((uint32_t)(q * 32) << 16);
            for (int c = 0; c < 8; ++c) {
                uint32_t r[32];
                tc_ld32(d + c * 32, r);
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = xt_act(__uint_as_float(r[i]), act);
                if (c == 7) {                                         // everything is in registers: hand the accumulator back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
                }
                const int col = col0 + c * 32;
                if (row < row_end && col < n) {
                    bf16* o = out + (size_t)row * n + col;
                    if (col + 32 <= n) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 p;
                            __nv_bfloat162 a0 = __floats2bfloat162_rn(v[i], v[i + 1]), a1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                            __nv_bfloat162 a2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), a3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                            p.x = *(uint32_t*)&a0; p.y = *(uint32_t*)&a1; p.z = *(uint32_t*)&a2; p.w = *(uint32_t*)&a3;
                            *(uint4*)(o + i) = p;
                        }
                    } else {
                        for (int i = 0; i < 32 && col + i < n; ++i) o[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * XT_BN) : "memory");
    }
}

static int xt_encode_map(CUtensorMap* map, const void* ptr, long rows, int k) {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {XT_BK, 128};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HB_REFUSE("expert_linear_tcgen05: cuTensorMapEncodeTiled failed with %d (rows %ld, k %d)", (int)r, rows, k);
    return 0;
}

HB_DEFINE_STATUS_MIRROR(hb_experts_tcgen05_status_mirror)
extern "C" int hb_experts_tcgen05_status(unsigned int* status) {
    HB_CUDA(cudaDeviceSynchronize());
    HB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned int)));
    const unsigned int zero = 0;
    HB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned int)));
    return 0;
}

extern "C" int hb_expert_linear_tcgen05_tiles(int rows, int experts) {
    return (rows + XT_BM - 1) / XT_BM + (experts < rows ? experts : rows);
}

// out [rows, n] = act(x' · w[e]ᵀ) for the rows of expert e (starts [experts + 1]); x' = x gathered by token_of into
// `gathered` [rows, k] (token_of null: x itself, its rows already expert by expert). table: 3 * hb_expert_linear_tcgen05_tiles
// (rows, experts) int32 of scratch. bfloat16; k and n multiples of 8; pointers 16-byte aligned.
extern "C" int hb_expert_linear_tcgen05(void* out, const void* x, const int32_t* token_of, void* gathered, const void* w,
                                        const int32_t* starts, int32_t* table, int rows, int experts, int n, int k, int act,
                                        hb_stream stream) {
    if (rows == 0 || n == 0) return 0;
    if (k < 8 || k % 8 || n % 8) HB_REFUSE("expert_linear_tcgen05: k = %d and n = %d must be multiples of 8", k, n);
    if (token_of && !gathered) HB_REFUSE("expert_linear_tcgen05: rows that are gathered need room for the gathered copy");
    const void* xs = token_of ? gathered : x;
    if ((((uintptr_t)xs | (uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16) != 0) HB_REFUSE("expert_linear_tcgen05: pointers must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const int tiles_m = hb_expert_linear_tcgen05_tiles(rows, experts);
    const int tiles_n = (n + XT_BN - 1) / XT_BN;
    expert_tiles_kernel<<<1, 32, 0, s>>>(table, starts, experts, tiles_m);
    HB_LAUNCH_CHECK("expert_tiles");
    if (token_of) {
        gather_rows_kernel<<<rows, 128, 0, s>>>((bf16*)gathered, (const bf16*)x, token_of, k);
        HB_LAUNCH_CHECK("gather_rows");
    }
    CUtensorMap map_x, map_w;
    int rc = xt_encode_map(&map_x, xs, rows, k);
    if (rc) return rc;
    rc = xt_encode_map(&map_w, w, (long)experts * n, k);
    if (rc) return rc;
    HB_CUDA(cudaFuncSetAttribute(expert_linear_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, XT_SMEM));
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        HB_CUDA(cudaGetDevice(&device));
        HB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    const long tiles = (long)tiles_m * tiles_n;
    const int grid = (int)(tiles < sms ? tiles : sms);
    expert_linear_tcgen05_kernel<<<grid, 192, XT_SMEM, s>>>(map_x, map_w, (bf16*)out, table, n, k, act, tiles_m, tiles_n);
    HB_LAUNCH_CHECK("expert_linear_tcgen05");
    return 0;
}
