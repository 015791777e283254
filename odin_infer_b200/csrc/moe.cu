// Mixture of experts on the CUDA cores: the router, and the experts' two products for the rows
// (token, choice) with each row reading the weights of its own expert.
//
//   router:   z = W_r h + b in 32-bit; the `top` largest logits are chosen (the lower index wins a tie),
//             their weights are the softmax over the chosen logits alone; `always` further rows per
//             token name the experts E, E + 1, ... with weight 1 (experts that every token uses).
//             score 1: the scores are sigmoid(z); the experts form `groups` equal groups of neighbours, a group's score
//             is the sum of its two largest scores, only experts of the `keep` best groups can be chosen; the weights are
//             the chosen scores divided by their sum (+ 1e-20), times `route_scale`.  With a gate row (row E of the
//             router's matrix) the `always` rows are weighted by sigmoid(row E . h), which also goes to `gate_out`.
//             score 2: the scores are the softmax over all rows of the router; an expert is chosen by score + correction (the
//             bias), a group's score is its largest choice score, and the weights are the chosen experts' scores (without the
//             correction) divided by their sum (+ 1e-20), times `route_scale`.  Rows from `n_real` on have no expert behind
//             them: a token that chooses one gets its own input back, times the weight (summed per token into `pass_out`).
//   gate|up:  a[r, j] = act(Wg[e_r] h_t)_j * (Wu[e_r] h_t)_j          r = t * rows_per_token + k
//             (not gated: a[r, j] = act(Wu[e_r] h_t)_j)
//   down:     y[k, t, :] = weight_r * Wd[e_r] a[r, :]                 32-bit, one slice per choice
//
// The slices y[k] are partial sums of the layer's update: whoever adds the update adds them in the
// order k = 0, 1, ...  Every sum runs in an order fixed by the sizes alone (a warp per output element,
// lanes striding the row), so a token's values do not depend on the batch.  These kernels serve the
// 32-bit path and steps of few tokens; rows of padding (sequence -1) get expert -1 and write zeros.
#include "common.cuh"
#include <math_constants.h>

#define MOE_THREADS 256
#define MOE_WARPS (MOE_THREADS / 32)
#define MOE_COLS 64  // output columns per block

#define MOE_ACT_SILU 1
#define MOE_ACT_GELU_TANH 2
#define MOE_ACT_RELU2 4

__device__ __forceinline__ float moe_activate(int act, float z) {
    if (act == MOE_ACT_SILU) return z / (1.0f + expf(-z));
    if (act == MOE_ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// sum_i w[i] x[i] over a row of n elements: lanes stride the row four vectors at a time (their loads go out together),
// the warp adds up; every lane gets the sum.  The order of the additions depends on n alone.
__device__ __forceinline__ float warp_dot(const float* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.f;
    if ((n & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int i0 = lane * 4; i0 < n; i0 += 512) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i0 + u * 128 < n) v[u] = *reinterpret_cast<const float4*>(w + i0 + u * 128);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * 128;
                if (i < n) {
                    acc = fmaf(v[u].x, x[i], acc);
                    acc = fmaf(v[u].y, x[i + 1], acc);
                    acc = fmaf(v[u].z, x[i + 2], acc);
                    acc = fmaf(v[u].w, x[i + 3], acc);
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(w[i], x[i], acc);
    }
    return warp_sum(acc);
}

__device__ __forceinline__ float warp_dot(const bf16* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.f;
    if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int i0 = lane * 8; i0 < n; i0 += 1024) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i0 + u * 256 < n) v[u] = *reinterpret_cast<const uint4*>(w + i0 + u * 256);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * 256;
                if (i < n) {
                    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(p[j]);
                        acc = fmaf(f.x, x[i + 2 * j], acc);
                        acc = fmaf(f.y, x[i + 2 * j + 1], acc);
                    }
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), x[i], acc);
    }
    return warp_sum(acc);
}

// ------------------------------------------------------------ router
// One block per token.  ids, wts: [T, top + always].  logits (optional): W h as a product has left it, float32 [T, E];
// the block then only adds the bias, chooses and weighs.
template <typename TH, typename TW>
__global__ void __launch_bounds__(1024)
moe_router_kernel(const TH* __restrict__ h, size_t h_stride, const TW* __restrict__ w, VecRef bias, int E, int d, int top,
                  int always, const int* __restrict__ tok_seq, int* __restrict__ ids, float* __restrict__ wts,
                  const float* __restrict__ logits, int score, int groups, int keep, float route_scale, int gate_row,
                  float* __restrict__ gate_out, int n_real, float* __restrict__ pass_out) {
    extern __shared__ float sm[];
    float* hrow = sm;       // d
    float* z = sm + d;      // E (+ 1 with a gate row)
    float* sc = z + E + 1;  // E: score 2 keeps the scores beside the choice scores
    const int rows = E + (gate_row ? 1 : 0);
    pdl_trigger();
    const int t = blockIdx.x, per = top + always;
    const bool real = tok_seq == nullptr || tok_seq[t] >= 0;
    pdl_wait();
    if (!real) {
        for (int k = threadIdx.x; k < per; k += blockDim.x) {
            ids[(size_t)t * per + k] = -1;
            wts[(size_t)t * per + k] = 0.f;
        }
        if (gate_out != nullptr && threadIdx.x == 0) gate_out[t] = 0.f;
        if (pass_out != nullptr && threadIdx.x == 0) pass_out[t] = 0.f;
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    if (logits != nullptr) {
        for (int e = threadIdx.x; e < rows; e += blockDim.x)
            z[e] = logits[(size_t)t * rows + e] + (bias.p != nullptr && e < E && score != 2 ? bias.at(e) : 0.f);
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) hrow[i] = to_f32(h[(size_t)t * h_stride + i]);
        __syncthreads();
        for (int e = warp; e < rows; e += n_warps) {
            const float s = warp_dot(w + (size_t)e * d, hrow, d, lane);
            if (lane == 0) z[e] = s + (bias.p != nullptr && e < E && score != 2 ? bias.at(e) : 0.f);
        }
    }
    __syncthreads();
    if (warp == 0) {
        float always_w = 1.0f;
        if (gate_row) {
            always_w = 1.0f / (1.0f + expf(-z[E]));
            if (gate_out != nullptr && lane == 0) gate_out[t] = always_w;
        }
        if (score == 1) {
            for (int e = lane; e < E; e += 32) z[e] = 1.0f / (1.0f + expf(-z[e]));
            __syncwarp();
            if (groups > 1) {
                // lane g: the sum of the two largest scores of group g; `keep` rounds of a warp-wide arg max
                // (the lower group wins a tie) mark the groups whose experts stay
                const int gsz = E / groups;
                float gs = -CUDART_INF_F;
                if (lane < groups) {
                    float a = -CUDART_INF_F, b = -CUDART_INF_F;
                    for (int e = lane * gsz; e < (lane + 1) * gsz; ++e) {
                        const float v = z[e];
                        if (v > a) { b = a; a = v; } else if (v > b) b = v;
                    }
                    gs = gsz > 1 ? a + b : a;
                }
                unsigned kept = 0u;
                for (int k = 0; k < keep; ++k) {
                    float best = gs;
                    int best_g = lane < groups ? lane : 0x7fffffff;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                        if (ov > best || (ov == best && og < best_g)) { best = ov; best_g = og; }
                    }
                    if (best_g < groups) kept |= 1u << best_g;
                    if (lane == best_g) gs = -CUDART_INF_F;
                }
                for (int e = lane; e < E; e += 32)
                    if (!((kept >> (e / gsz)) & 1u)) z[e] = -CUDART_INF_F;
                __syncwarp();
            }
        }
        if (score == 2) {
            // scores: the softmax over all rows; choice scores: score + correction (the bias); a group's score is its
            // largest choice score; the groups that do not stay count as minus infinity
            float m = -CUDART_INF_F;
            for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
            m = warp_max(m);
            float tot = 0.f;
            for (int e = lane; e < E; e += 32) { const float pe = expf(z[e] - m); sc[e] = pe; tot += pe; }
            tot = warp_sum(tot);
            for (int e = lane; e < E; e += 32) {
                const float se = sc[e] / tot;
                sc[e] = se;
                z[e] = se + (bias.p != nullptr ? bias.at(e) : 0.f);
            }
            __syncwarp();
            if (groups > 1) {
                const int gsz = E / groups;
                float gs = -CUDART_INF_F;
                if (lane < groups)
                    for (int e = lane * gsz; e < (lane + 1) * gsz; ++e) gs = fmaxf(gs, z[e]);
                unsigned kept = 0u;
                for (int k = 0; k < keep; ++k) {
                    float best = gs;
                    int best_g = lane < groups ? lane : 0x7fffffff;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                        if (ov > best || (ov == best && og < best_g)) { best = ov; best_g = og; }
                    }
                    if (best_g < groups) kept |= 1u << best_g;
                    if (lane == best_g) gs = -CUDART_INF_F;
                }
                for (int e = lane; e < E; e += 32)
                    if (!((kept >> (e / gsz)) & 1u)) z[e] = -CUDART_INF_F;
                __syncwarp();
            }
        }
        // `top` rounds of a warp-wide arg max; the chosen logit is taken out by -inf
        float chosen = 0.f, first = 0.f, sum = 0.f;
        int chosen_id = -1;
        for (int k = 0; k < top; ++k) {
            float best = -CUDART_INF_F;
            int best_e = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = z[e];
                if (v > best) { best = v; best_e = e; }  // ascending e: the lower index stays on a tie
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
            }
            if (k == 0) first = best;
            const float p = score == 1 ? best : score == 2 ? (best_e < E ? sc[best_e] : 0.f) : expf(best - first);
            sum += p;
            if (lane == k) { chosen = p; chosen_id = best_e; }
            if (lane == 0 && best_e < E) z[best_e] = -CUDART_INF_F;
            __syncwarp();
        }
        // rows from n_real on have no expert behind them: their weights are summed into pass_out (the token's input is
        // handed through that many times) and their places name no expert
        const float wt = score != 0 ? chosen / (sum + 1e-20f) * route_scale : chosen / sum;
        const bool passes = lane < top && chosen_id >= n_real && chosen_id < E;
        const float passed = warp_sum(passes ? wt : 0.f);
        if (pass_out != nullptr && lane == 0) pass_out[t] = passed;
        if (lane < top) {
            ids[(size_t)t * per + lane] = chosen_id < n_real ? chosen_id : -1;
            wts[(size_t)t * per + lane] = passes ? 0.f : wt;
        }
        for (int k = lane; k < always; k += 32) {
            ids[(size_t)t * per + top + k] = n_real + k;
            wts[(size_t)t * per + top + k] = always_w;
        }
    }
}

extern "C" int odin_moe_router(const void* h, int h_dtype, long long h_stride, const void* w, int w_dtype, const void* bias,
                               int bias_dtype, int T, int E, int d, int top, int always, const int* tok_seq, int* ids,
                               float* wts, const float* logits, int score, int groups, int keep, float route_scale,
                               int gate_row, float* gate_out, int n_real, float* pass_out, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > 32 || top > E || always < 0 || d <= 0) return ODIN_ERR_UNSUPPORTED;
    if (score < 0 || score > 2 || n_real < 0 || n_real > E || (n_real < E && pass_out == nullptr)) return ODIN_ERR_BAD_ARG;
    if (groups < 1 || groups > 32 || E % groups != 0 || keep < 1 || keep > groups || (long long)keep * (E / groups) < top)
        return ODIN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(d + 2 * E + 1) * sizeof(float);
    if (smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef bv{bias, bias_dtype == ODIN_BF16};
    // a warp per expert while the tokens are few (their blocks cannot fill the GPU); four warps a token else
    int threads = 128;
    if (logits != nullptr) threads = 32;
    else if (T <= 64) threads = E >= 32 ? 1024 : E >= 16 ? 512 : E >= 8 ? 256 : 128;
#define GO(TH, TW)                                                                                                   \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(moe_router_kernel<TH, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        odin_launch(moe_router_kernel<TH, TW>, dim3(T), dim3(threads), smem, s, (const TH*)h, (size_t)h_stride,      \
                    (const TW*)w, bv, E, d, top, always, tok_seq, ids, wts, logits, score, groups, keep,             \
                    route_scale, gate_row, gate_out, n_real, pass_out);                                              \
    } while (0)
    if (h_dtype == ODIN_BF16 && w_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (h_dtype == ODIN_F32 && w_dtype == ODIN_F32) GO(float, float);
    else if (h_dtype == ODIN_BF16 && w_dtype == ODIN_F32) GO(bf16, float);
    else if (h_dtype == ODIN_F32 && w_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ gate|up of the rows' own experts
// grid (rows, column blocks).  w: [experts][2 ff][d], the ff gate rows before the ff up rows (not gated: [experts][ff][d]).
template <typename TH, typename TW>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(const TH* __restrict__ h, size_t h_stride, const TW* __restrict__ w, const int* __restrict__ ids, int per,
                   int ff, int d, int act, int gated, TH* __restrict__ out) {
    extern __shared__ float hrow[];  // d
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, t = r / per;
    const int e = ids[r];
    const int c0 = blockIdx.y * MOE_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TH* orow = out + (size_t)r * ff;
    if (e < 0) {
        for (int j = c0 + threadIdx.x; j < min(ff, c0 + MOE_COLS); j += blockDim.x) orow[j] = from_f32<TH>(0.f);
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) hrow[i] = to_f32(h[(size_t)t * h_stride + i]);
    __syncthreads();
    const TW* we = w + (size_t)e * (gated ? 2 : 1) * ff * d;
    for (int j = c0 + warp; j < min(ff, c0 + MOE_COLS); j += MOE_WARPS) {
        const float g = warp_dot(we + (size_t)j * d, hrow, d, lane);
        const float u = gated ? warp_dot(we + (size_t)(ff + j) * d, hrow, d, lane) : 1.0f;
        if (lane == 0) orow[j] = from_f32<TH>(gated ? moe_activate(act, g) * u : moe_activate(act, g));
    }
}

extern "C" int odin_moe_gate_up(const void* h, int h_dtype, long long h_stride, const void* w, int w_dtype, const int* ids,
                                int T, int per, int ff, int d, int act, int gated, void* out, void* stream) {
    if (T <= 0 || per <= 0) return 0;
    if (act != MOE_ACT_SILU && act != MOE_ACT_GELU_TANH && act != MOE_ACT_RELU2) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024 || (long long)T * per > 2147483647LL) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)(T * per), (unsigned)((ff + MOE_COLS - 1) / MOE_COLS));
#define GO(TH, TW)                                                                                                    \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(moe_gate_up_kernel<TH, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        odin_launch(moe_gate_up_kernel<TH, TW>, grid, dim3(MOE_THREADS), smem, s, (const TH*)h, (size_t)h_stride,     \
                    (const TW*)w, ids, per, ff, d, act, gated, (TH*)out);                                             \
    } while (0)
    if (h_dtype == ODIN_BF16 && w_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (h_dtype == ODIN_F32 && w_dtype == ODIN_F32) GO(float, float);
    else if (h_dtype == ODIN_BF16 && w_dtype == ODIN_F32) GO(bf16, float);
    else if (h_dtype == ODIN_F32 && w_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ down product of the rows' own experts, weighted
// a: [T * per, ff]; w: [experts][d][ff]; y: [per][T][d] 32-bit, y[k][t] = wts[t, k] * Wd[e] a[t * per + k]
template <typename TA, typename TW>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(const TA* __restrict__ a, const TW* __restrict__ w, const int* __restrict__ ids, const float* __restrict__ wts,
                int T, int per, int ff, int d, float* __restrict__ y) {
    extern __shared__ float arow[];  // ff
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, t = r / per, k = r % per;
    const int e = ids[r];
    const int c0 = blockIdx.y * MOE_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* yrow = y + ((size_t)k * T + t) * d;
    if (e < 0) {
        for (int c = c0 + threadIdx.x; c < min(d, c0 + MOE_COLS); c += blockDim.x) yrow[c] = 0.f;
        return;
    }
    for (int i = threadIdx.x; i < ff; i += blockDim.x) arow[i] = to_f32(a[(size_t)r * ff + i]);
    __syncthreads();
    const float wt = wts[r];
    const TW* we = w + (size_t)e * d * ff;
    for (int c = c0 + warp; c < min(d, c0 + MOE_COLS); c += MOE_WARPS) {
        const float s = warp_dot(we + (size_t)c * ff, arow, ff, lane);
        if (lane == 0) yrow[c] = wt * s;
    }
}

extern "C" int odin_moe_down(const void* a, int a_dtype, const void* w, int w_dtype, const int* ids, const float* wts, int T,
                             int per, int ff, int d, float* y, void* stream) {
    if (T <= 0 || per <= 0) return 0;
    const size_t smem = (size_t)ff * sizeof(float);
    if (smem > 200 * 1024 || (long long)T * per > 2147483647LL) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)(T * per), (unsigned)((d + MOE_COLS - 1) / MOE_COLS));
#define GO(TA, TW)                                                                                                 \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(moe_down_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        odin_launch(moe_down_kernel<TA, TW>, grid, dim3(MOE_THREADS), smem, s, (const TA*)a, (const TW*)w, ids,    \
                    wts, T, per, ff, d, y);                                                                        \
    } while (0)
    if (a_dtype == ODIN_BF16 && w_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (a_dtype == ODIN_F32 && w_dtype == ODIN_F32) GO(float, float);
    else if (a_dtype == ODIN_BF16 && w_dtype == ODIN_F32) GO(bf16, float);
    else if (a_dtype == ODIN_F32 && w_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}
