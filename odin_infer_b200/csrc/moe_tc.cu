// Experts chosen per token, for many tokens: the rows (token, choice) are put in the order of their experts, each
// expert's rows padded to whole tiles of 128, and the two products run as grouped matrix products on the tcgen05
// tensor cores: every output tile multiplies 128 sorted rows with the weight rows of that tile's own expert.
//
//   plan      counts the rows of every expert, gives every row its place in the sorted order and every tile of
//             128 places its expert (-1: no rows), and lists for every place the row it holds (-1: padding);
//   gather    a_sorted[place] = h[row / per] (bfloat16), zeros in padding;
//   grouped   C[place, :] = act(A Wg[e]^T) * (A Wu[e]^T)  (DUAL: gate and up accumulators side by side in tensor
//             memory, the activation applied as they are read back), or C[place, :] = A W[e]^T in 32-bit;
//   combine   y[t, :] = sum_k wts[t, k] * C[place(t, k), :], the choices in their order: the tokens' update.
//
// A row's values do not depend on its place (each output element is its own sum over K in the order of the K
// blocks), so the places may be handed out in any order: equal inputs give equal bits whatever the batch.
// The grouped kernel: one CTA per (column tile, row tile); warp 0 feeds a ring of stages by TMA (128-byte swizzle),
// one lane of warp 1 issues the MMAs (128 x 256 each) into tensor memory, warps 2..5 read the accumulator back and
// store.  With many tiles two CTAs share an SM, so one's epilogue runs beside the other's products; with few, each has
// a longer ring.  Every wait is bounded (tc::mbar_wait).
#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace {

constexpr int BM = 128;   // sorted rows per tile (MMA M)
constexpr int BN = 128;   // output columns per accumulator of the gated product (MMA N); the plain product takes 2 BN
constexpr int BK = 64;    // K elements per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;

#define MOE_ACT_SILU 1
#define MOE_ACT_GELU_TANH 2
#define MOE_ACT_RELU2 4

// ------------------------------------------------------------------------------------------------ plan
// One CTA.  ids: [rows] expert of every row (-1: none).  Outputs: place_of_row [rows] (-1: none), row_of_place
// [places_cap] (-1: padding), tile_expert [places_cap / 128] (-1: unused).
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int rows, int n_experts, int* __restrict__ place_of_row,
                int* __restrict__ row_of_place, int places_cap, int* __restrict__ tile_expert) {
    extern __shared__ int sm[];
    int* count = sm;                   // [n_experts]
    int* first = sm + n_experts;       // [n_experts] first place of the expert
    int* cursor = sm + 2 * n_experts;  // [n_experts]
    pdl_trigger();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    pdl_wait();
    for (int i = threadIdx.x; i < places_cap; i += blockDim.x) row_of_place[i] = -1;
    for (int i = threadIdx.x; i < places_cap / BM; i += blockDim.x) tile_expert[i] = -1;
    // a thread's rows are loaded together (a loop of load, atomic, load, ... is a chain of memory latencies); rows
    // beyond PLAN_HELD per thread are read again in the second pass
    constexpr int PLAN_HELD = 16;
    int held[PLAN_HELD];
#pragma unroll
    for (int k = 0; k < PLAN_HELD; ++k) {
        const int r = threadIdx.x + k * 1024;
        held[k] = r < rows ? ids[r] : -1;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < PLAN_HELD; ++k)
        if (held[k] >= 0 && held[k] < n_experts) atomicAdd(&count[held[k]], 1);
    for (int r = threadIdx.x + PLAN_HELD * 1024; r < rows; r += 1024) {
        const int e = ids[r];
        if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = at;
            at += (count[e] + BM - 1) / BM * BM;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        for (int t = first[e] / BM; t < (first[e] + count[e] + BM - 1) / BM; ++t) tile_expert[t] = e;
#pragma unroll
    for (int k = 0; k < PLAN_HELD; ++k) {
        const int r = threadIdx.x + k * 1024;
        if (r < rows) {
            const int e = held[k];
            int place = -1;
            if (e >= 0 && e < n_experts) {
                place = first[e] + atomicAdd(&cursor[e], 1);
                row_of_place[place] = r;
            }
            place_of_row[r] = place;
        }
    }
    for (int r = threadIdx.x + PLAN_HELD * 1024; r < rows; r += 1024) {
        const int e = ids[r];
        int place = -1;
        if (e >= 0 && e < n_experts) {
            place = first[e] + atomicAdd(&cursor[e], 1);
            row_of_place[place] = r;
        }
        place_of_row[r] = place;
    }
}

// ------------------------------------------------------------------------------------------------ gather
// A block takes GATHER_PLACES places; their row numbers, then their rows' loads go out together.
constexpr int GATHER_PLACES = 4;
__global__ void __launch_bounds__(256)
moe_gather_kernel(const bf16* __restrict__ h, size_t h_stride, const int* __restrict__ row_of_place, int places, int per, int d,
                  bf16* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int p0 = blockIdx.x * GATHER_PLACES;
    int r[GATHER_PLACES];
#pragma unroll
    for (int k = 0; k < GATHER_PLACES; ++k) r[k] = (p0 + k < places) ? row_of_place[p0 + k] : -2;
    for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
        uint4 v[GATHER_PLACES];
#pragma unroll
        for (int k = 0; k < GATHER_PLACES; ++k)
            v[k] = r[k] >= 0 ? *reinterpret_cast<const uint4*>(h + (size_t)(r[k] / per) * h_stride + i) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < GATHER_PLACES; ++k)
            if (r[k] != -2) *reinterpret_cast<uint4*>(out + (size_t)(p0 + k) * d + i) = v[k];
    }
}

// ------------------------------------------------------------------------------------------------ combine
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ c, const int* __restrict__ place_of_row, const float* __restrict__ wts, int per,
                   int d, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < per; ++k) {
            const int place = place_of_row[t * per + k];
            if (place < 0) continue;
            const float w = wts[t * per + k];
            const float4 v = *reinterpret_cast<const float4*>(c + (size_t)place * d + i);
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        *reinterpret_cast<float4*>(y + (size_t)t * d + i) = acc;
    }
}

// ------------------------------------------------------------------------------------------------ grouped product
struct GroupedParams {
    void* out;
    long long ldc;
    int N;                 // output columns (DUAL: the inner size)
    int K;
    int rows_per_expert;   // weight rows of one expert in the stacked matrix (DUAL: 2 N, gate rows first)
    int act;
    int stages;            // length of the ring of stages (2: two CTAs share an SM; 4: few CTAs, each with more in flight)
    const int* tile_expert;
    int* error;
};

// DUAL: two accumulators of BN columns (gate, up), two weight boxes of BN rows a stage.  Plain: one accumulator of
// 2 BN columns, one weight box of 2 BN rows.  Either way a stage is 48 KB and the CTA holds 256 columns.
struct GCfg {
    static constexpr int MAX_STAGES = 4;
    static constexpr int STAGE_A = BM * BK * 2;
    static constexpr int STAGE_B = 2 * BN * BK * 2;
    static constexpr int STAGE = STAGE_A + STAGE_B;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int HEAD = 1024;  // barriers and flags, before the stages (which start 1024-byte aligned)
    static constexpr int smem(int stages) { return 1024 + HEAD + stages * STAGE; }
};

__device__ __forceinline__ float act_gate(int act, float g) {
    if (act == MOE_ACT_SILU) return __fdividef(g, 1.0f + __expf(-g));
    const float y2 = 1.5957691216057308f * g * fmaf(0.044715f * g, g, 1.0f);   // g sigmoid(2 y) = tanh-GELU
    return __fdividef(g, 1.0f + __expf(-y2));
}

// an expert without a gate matrix: the activation of its one accumulator (relu2: max(z, 0)^2)
__device__ __forceinline__ float act_alone(int act, float z) {
    if (act == MOE_ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    return act_gate(act, z);
}

template <bool DUAL, typename TO>
__global__ void __launch_bounds__(192)
moe_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const GroupedParams p) {
    using C = GCfg;
    constexpr int TILE_N = DUAL ? BN : 2 * BN;   // output columns of a tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(base);
    uint64_t* empty = full + C::MAX_STAGES;
    uint64_t* acc_full = empty + C::MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* smem = base + 1024;   // the stages: 1024-byte aligned for the 128-byte swizzle
    const uint32_t n_stages = (uint32_t)p.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::MAX_STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
        tc::mbar_init(acc_full, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    pdl_wait();   // the plan, the sorted rows and the output's memory belong to earlier kernels until here
    const int tile_m = blockIdx.y, tile_n = blockIdx.x;
    const int e = p.tile_expert[tile_m];
    if (e < 0) return;   // a tile of places that no expert's rows reach (the whole CTA leaves, nothing is held yet)
    if (warp == 1) tc::tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int n_kb = (p.K + BK - 1) / BK;
    const int w_row0 = e * p.rows_per_expert + tile_n * TILE_N;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                uint8_t* sa = smem + stage * C::STAGE;
                tc::mbar_expect_tx(&full[stage], C::STAGE);
                tc::tma_load_2d(sa, &map_a, kb * BK, tile_m * BM, &full[stage]);
                if (DUAL) {   // two boxes of BN rows: the gate rows and, N rows further, the up rows
                    tc::tma_load_2d(sa + C::STAGE_A, &map_w, kb * BK, w_row0, &full[stage]);
                    tc::tma_load_2d(sa + C::STAGE_A + C::STAGE_B / 2, &map_w, kb * BK, w_row0 + p.N, &full[stage]);
                } else {      // one box of 2 BN rows
                    tc::tma_load_2d(sa + C::STAGE_A, &map_w, kb * BK, w_row0, &full[stage]);
                }
                if (++stage == n_stages) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                // aborted: let the copies already in flight land before the CTA's memory is released
                for (uint32_t s2 = 0; s2 < n_stages; ++s2)
                    for (uint32_t i = 0; i < 4096; ++i)
                        if (tc::mbar_try_wait(&full[s2], 0) || tc::mbar_try_wait(&full[s2], 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // the gate and up tiles lie one after the other in a stage: one MMA of 2 BN columns covers both
            // accumulators (DUAL) or the one wide accumulator (plain)
            constexpr uint32_t idesc = tc::make_idesc_bf16(BM, 2 * BN);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int kb = 0; kb < n_kb; ++kb) {
                if (!tc::mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t ax = tc::smem_u32(smem + stage * C::STAGE);
                const uint64_t da = tc::make_smem_desc_sw128(ax);
                const uint64_t db = tc::make_smem_desc_sw128(ax + C::STAGE_A);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)   // +32 bytes per K step inside the swizzle row: +2 in 16-byte units
                    tc::umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                tc::umma_commit(&empty[stage]);
                if (++stage == n_stages) { stage = 0; phase ^= 1; }
            }
            if (ok) tc::umma_commit(acc_full);
        }
    } else {
        const int quarter = warp & 3;   // the tensor-memory lanes this warp may read: [32 quarter, +32)
        if (tc::mbar_wait(acc_full, 0, abort_flag)) {
            tc::fence_after_sync();
            const size_t i = (size_t)tile_m * BM + quarter * 32 + lane;   // the place; every place of a tile exists
            TO* out = reinterpret_cast<TO*>(p.out) + i * p.ldc;
#pragma unroll 1
            for (int c0 = 0; c0 < TILE_N; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + c0;
                if (DUAL) {
                    uint32_t u[32];
                    tc::tmem_ld32(taddr, r);
                    tc::tmem_ld32(taddr + BN, u);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(act_gate(p.act, __uint_as_float(r[q])) * __uint_as_float(u[q]));
                } else {
                    tc::tmem_ld32(taddr, r);
                    tc::tmem_ld_wait();
                    if (p.act != 0) {
#pragma unroll
                        for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(act_alone(p.act, __uint_as_float(r[q])));
                    }
                }
                const int j0 = tile_n * TILE_N + c0;
                if (j0 < p.N) {
                    const int n = min(32, p.N - j0);
                    if (sizeof(TO) == 4) {
                        float* dst = reinterpret_cast<float*>(out) + j0;
                        if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
                            for (int q = 0; q < n; ++q) dst[q] = __uint_as_float(r[q]);
                        }
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(out) + j0;
                        if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t w[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * j]), __uint_as_float(r[8 * q + 2 * j + 1]));
                                    w[j] = *reinterpret_cast<uint32_t*>(&hh);
                                }
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
                            for (int q = 0; q < n; ++q) dst[q] = __float2bfloat16_rn(__uint_as_float(r[q]));
                        }
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error != nullptr) atomicCAS(p.error, 0, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// A row-major [rows, K] bfloat16 matrix with row stride ld, read in boxes of 64 (K) x box_rows rows, 128-byte
// swizzle, zeros beyond the edges.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return ODIN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ODIN_ERR_BAD_ARG;
}

int* error_flag() {
    static int* flag = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&flag, sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, sizeof(int));
        else flag = nullptr;
    });
    return flag;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <bool DUAL, typename TO>
int launch_grouped(const CUtensorMap& ma, const CUtensorMap& mw, GroupedParams p, int tiles_m, cudaStream_t s) {
    using C = GCfg;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<DUAL, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::smem(C::MAX_STAGES));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tile_n = DUAL ? BN : 2 * BN;
    const dim3 grid((unsigned)((p.N + tile_n - 1) / tile_n), (unsigned)tiles_m);
    // Few CTAs (a step of few tokens: the weights stream once, and about half of the grid's row tiles are places that no
    // expert's rows reach, whose CTAs leave at once; measured at 138 working CTAs: 37.5 us against 43.6): a ring of four
    // stages, so that enough is in flight; many CTAs: two stages, and two CTAs share an SM, one's epilogue beside the
    // other's products.  The number of CTAs follows from the shapes alone.
    p.stages = ((long long)grid.x * grid.y <= 2LL * sm_count()) ? C::MAX_STAGES : 2;
    odin_launch(moe_grouped_kernel<DUAL, TO>, grid, dim3(192), (size_t)C::smem(p.stages), s, ma, mw, p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// Places that `rows` rows of `n_experts` experts can take at most (a multiple of 128).
extern "C" long long odin_moe_places(long long rows, int n_experts) {
    return (rows + (long long)n_experts * (BM - 1) + BM - 1) / BM * BM;
}

extern "C" int odin_moe_plan(const int* ids, int rows, int n_experts, int* place_of_row, int* row_of_place, int places_cap,
                             int* tile_expert, void* stream) {
    if (rows <= 0) return 0;
    if (n_experts <= 0 || n_experts > 4096 || places_cap % BM != 0 || places_cap < odin_moe_places(rows, n_experts))
        return ODIN_ERR_BAD_ARG;
    odin_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)3 * n_experts * sizeof(int), (cudaStream_t)stream, ids, rows,
                n_experts, place_of_row, row_of_place, places_cap, tile_expert);
    ODIN_LAUNCH_CHECK();
    return 0;
}

extern "C" int odin_moe_gather(const void* h, long long h_stride, const int* row_of_place, int places, int per, int d, void* out,
                               void* stream) {
    if (places <= 0) return 0;
    if (d % 8 != 0 || h_stride % 8 != 0 || ((((uintptr_t)h) | ((uintptr_t)out)) & 15) != 0) return ODIN_ERR_UNSUPPORTED;
    odin_launch(moe_gather_kernel, dim3((places + GATHER_PLACES - 1) / GATHER_PLACES), dim3(256), 0, (cudaStream_t)stream,
                (const bf16*)h, (size_t)h_stride, row_of_place, places, per, d, (bf16*)out);
    ODIN_LAUNCH_CHECK();
    return 0;
}

extern "C" int odin_moe_combine(const float* c, const int* place_of_row, const float* wts, int T, int per, int d, float* y,
                                void* stream) {
    if (T <= 0) return 0;
    if (d % 4 != 0 || ((((uintptr_t)c) | ((uintptr_t)y)) & 15) != 0) return ODIN_ERR_UNSUPPORTED;
    odin_launch(moe_combine_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, c, place_of_row, wts, per, d, y);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// a: [places, K] bfloat16 sorted rows; w: [experts * rows_per_expert, K] bfloat16, the experts' matrices stacked.
// dual = 1: rows_per_expert = 2 N (N gate rows, then N up rows), out[places, N] = act(a Wg^T) * (a Wu^T), bfloat16;
// dual = 0: rows_per_expert = N, out[places, N] = a W^T in 32-bit (act = 0), or act(a W^T) in bfloat16 (silu, gelu_tanh, relu2).
extern "C" int odin_moe_grouped(const void* a, long long lda, const void* w, long long ldw, int n_experts, int rows_per_expert,
                                int places, int N, int K, int dual, int act, const int* tile_expert, void* out, long long ldc,
                                void* stream) {
    if (places <= 0 || N <= 0) return 0;
    if (places % BM != 0 || K <= 0 || rows_per_expert != (dual ? 2 * N : N)) return ODIN_ERR_BAD_ARG;
    if (dual && act != MOE_ACT_SILU && act != MOE_ACT_GELU_TANH) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)a) & 15) || (((uintptr_t)w) & 15)) return ODIN_ERR_UNSUPPORTED;
    CUtensorMap ma, mw;
    int rc;
    if ((rc = make_map(&ma, a, places, K, lda, BM))) return rc;
    if ((rc = make_map(&mw, w, (long long)n_experts * rows_per_expert, K, ldw, dual ? BN : 2 * BN))) return rc;
    GroupedParams p;
    p.out = out; p.ldc = ldc; p.N = N; p.K = K; p.rows_per_expert = rows_per_expert; p.act = act; p.stages = 2;
    p.tile_expert = tile_expert;
    p.error = error_flag();
    cudaStream_t s = (cudaStream_t)stream;
    if (dual) return launch_grouped<true, bf16>(ma, mw, p, places / BM, s);
    if (act != 0) {
        if (act != MOE_ACT_SILU && act != MOE_ACT_GELU_TANH && act != MOE_ACT_RELU2) return ODIN_ERR_BAD_ARG;
        return launch_grouped<false, bf16>(ma, mw, p, places / BM, s);
    }
    return launch_grouped<false, float>(ma, mw, p, places / BM, s);
}

extern "C" int odin_moe_tc_error() {
    int* f = error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(f, 0, sizeof(int));
    return v;
}
