// State-space mixers: what stands around and inside a selective scan.
//
//   * causal convolution per channel over a sequence's rows, with a bias and an optional SiLU; the rows before a
//     step's first one come from the sequence's state (its last taps - 1 inputs, zeros at a sequence's start), and a
//     second kernel stores the step's last inputs there;
//   * the selective scan with one state row per channel:
//         dt = softplus(raw + bias);  S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c
//     then y * silu(z);
//   * the tail of a scan with matrix-valued states per head (its recurrence is `linear_recurrence`'s): o + D_h x, times
//     silu(z), RMSNorm in equal consecutive parts of the row, times a weight.
//
// Step sizes, decays, exponentials and the state are 32-bit whatever the activations' type.  A sequence's tokens are
// walked in order by the threads that own a channel, so a token's values do not depend on how the tokens were cut into
// steps or on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ float ss_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float ss_silu(float z) { return z / (1.0f + expf(-z)); }

// ------------------------------------------------------------ causal convolution
// out[t, c] = act(b[c] + sum_j w[c, j] * in[t - (taps - 1 - j), c]); rows before the sequence's first row of this step
// are read from state[slot][taps - 1 - m][c] (m rows before).  grid (rows, channel blocks).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const TI* __restrict__ in, size_t in_stride, VecRef w, VecRef bias, int taps, int silu,
                   const float* __restrict__ state, size_t state_stride, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slots, TO* __restrict__ out,
                   size_t out_stride, int C) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int seq = tok_seq[t];
    int first = 0, slot = 0;
    if (seq >= 0) { first = seq_start[seq]; slot = seq_slots[seq]; }
    pdl_wait();
    if (seq < 0 || c >= C) return;
    float acc = bias.p != nullptr ? bias.at(c) : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int r = t - (taps - 1 - j);
        float v;
        if (r >= first) v = to_f32(in[(size_t)r * in_stride + c]);
        else v = state[(size_t)slot * state_stride + (size_t)(taps - 1 - (first - r)) * C + c];
        acc = fmaf(w.at(c * taps + j), v, acc);
    }
    out[(size_t)t * out_stride + c] = from_f32<TO>(silu ? ss_silu(acc) : acc);
}

// state[slot] <- the last taps - 1 inputs of (old state ++ the step's rows).  grid (sequences, channel blocks).
template <typename TI>
__global__ void __launch_bounds__(256)
conv_state_kernel(const TI* __restrict__ in, size_t in_stride, int taps, float* __restrict__ state, size_t state_stride,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_slots, int C) {
    pdl_trigger();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = seq_start[b], n_new = seq_start[b + 1] - first, slot = seq_slots[b];
    pdl_wait();
    if (n_new <= 0 || c >= C) return;
    float* st = state + (size_t)slot * state_stride + c;
    const int keep = taps - 1;
    for (int k = 0; k < keep; ++k) {   // ascending: an old value is read before its place is written
        const int p = n_new + k;       // place in (old state ++ new rows)
        st[(size_t)k * C] = p < keep ? st[(size_t)p * C] : to_f32(in[(size_t)(first + p - keep) * in_stride + c]);
    }
}

extern "C" int odin_causal_conv(const void* in, int in_dtype, long long in_stride, const void* w, int w_dtype,
                                const void* bias, int bias_dtype, int taps, int silu, float* state, long long state_stride,
                                const int* tok_seq, const int* seq_start, const int* seq_slots, int n_seqs, void* out,
                                int out_dtype, long long out_stride, int T, int C, void* stream) {
    if (T <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > 64 || n_seqs <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef wv{w, w_dtype == ODIN_BF16}, bv{bias, bias_dtype == ODIN_BF16};
    const int threads = C >= 256 ? 256 : (C + 31) / 32 * 32;
    dim3 grid(T, (C + threads - 1) / threads);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
#define GO(TI, TO)                                                                                                   \
    odin_launch(causal_conv_kernel<TI, TO>, grid, dim3(threads), 0, s, (const TI*)in, (size_t)in_stride, wv, bv, taps, \
                silu, (const float*)state, (size_t)state_stride, tok_seq, seq_start, seq_slots, (TO*)out,             \
                (size_t)out_stride, C)
    if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_F32) GO(bf16, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    if (taps > 1) {
        dim3 g2(n_seqs, grid.y);
        if (in_dtype == ODIN_BF16)
            odin_launch(conv_state_kernel<bf16>, g2, dim3(threads), 0, s, (const bf16*)in, (size_t)in_stride, taps, state,
                        (size_t)state_stride, seq_start, seq_slots, C);
        else
            odin_launch(conv_state_kernel<float>, g2, dim3(threads), 0, s, (const float*)in, (size_t)in_stride, taps, state,
                        (size_t)state_stride, seq_start, seq_slots, C);
        ODIN_LAUNCH_CHECK();
    }
    return 0;
}

// ------------------------------------------------------------ selective scan, a state row per channel
// A CTA owns SCAN_CH channels of one sequence; SCAN_LANES neighbouring lanes share a channel, lane l holding the state
// indices l, l + SCAN_LANES, ... in registers (NPL of them).  A block of tokens' inputs is staged in shared memory (the
// step size with its softplus taken once per token and channel); a token then costs a thread NPL exponentials and 2 NPL
// multiply-adds, and the channel's output is the sum of its lanes' shares (two shuffles, always in the same order).
#define SCAN_LANES 4
#define SCAN_CH 32
#define SCAN_TOK 16
struct ScanParams {
    const void* x; int x_is_bf16; long long x_stride;       // [rows, inner] (after the convolution and its activation)
    const float* dt; long long dt_stride; VecRef dt_bias;   // raw step sizes [rows, inner]
    const float* B; const float* C; long long bc_stride;    // [rows, N] each
    VecRef A_log, D;                                        // [inner, N], [inner]
    const void* z; long long z_stride;                      // gate [rows, inner], element type of x (null: none)
    float* state; long long state_stride;                   // per slot [inner][N]
    void* out; int out_is_bf16; long long out_stride;
    const int* seq_start; const int* seq_slots;
    int inner, N;
};

template <int NPL>
__global__ void __launch_bounds__(SCAN_CH * SCAN_LANES)
selective_scan_kernel(ScanParams p) {
    extern __shared__ float scan_sm[];
    const int N = p.N;
    float* sB = scan_sm;                       // [SCAN_TOK][N]
    float* sC = sB + SCAN_TOK * N;             // [SCAN_TOK][N]
    float* sx = sC + SCAN_TOK * N;             // [SCAN_TOK][SCAN_CH]
    float* sdt = sx + SCAN_TOK * SCAN_CH;
    float* sz = sdt + SCAN_TOK * SCAN_CH;
    pdl_trigger();
    const int b = blockIdx.x, ch0 = blockIdx.y * SCAN_CH;
    const int cl = threadIdx.x / SCAN_LANES, l = threadIdx.x % SCAN_LANES;
    const int c = ch0 + cl;
    const bool live = c < p.inner;
    const int row0 = p.seq_start[b], row1 = p.seq_start[b + 1], slot = p.seq_slots[b];
    float A[NPL], S[NPL];
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        A[j] = (live && n < N) ? -expf(p.A_log.at(c * N + n)) : 0.f;
    }
    const float Dc = (live && p.D.p != nullptr) ? p.D.at(c) : 0.f;
    pdl_wait();
    if (row1 <= row0) return;   // an empty (padding) sequence owns no state
    float* st = p.state + (size_t)slot * p.state_stride + (size_t)c * N;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        S[j] = (live && n < N) ? st[n] : 0.f;
    }
    for (int t0 = row0; t0 < row1; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, row1 - t0);
        __syncthreads();   // the block before has been walked
        for (int e = threadIdx.x; e < nt * N; e += blockDim.x) {
            const int u = e / N, n = e % N;
            sB[u * N + n] = p.B[(size_t)(t0 + u) * p.bc_stride + n];
            sC[u * N + n] = p.C[(size_t)(t0 + u) * p.bc_stride + n];
        }
        for (int e = threadIdx.x; e < nt * SCAN_CH; e += blockDim.x) {
            const int u = e / SCAN_CH, cc = ch0 + e % SCAN_CH;
            float xv = 0.f, dv = 0.f, zv = 0.f;
            if (cc < p.inner) {
                const size_t r = (size_t)(t0 + u);
                xv = p.x_is_bf16 ? __bfloat162float(((const bf16*)p.x)[r * p.x_stride + cc]) : ((const float*)p.x)[r * p.x_stride + cc];
                dv = ss_softplus(p.dt[r * p.dt_stride + cc] + (p.dt_bias.p != nullptr ? p.dt_bias.at(cc) : 0.f));
                if (p.z != nullptr)
                    zv = p.x_is_bf16 ? __bfloat162float(((const bf16*)p.z)[r * p.z_stride + cc]) : ((const float*)p.z)[r * p.z_stride + cc];
            }
            sx[e] = xv; sdt[e] = dv; sz[e] = zv;
        }
        __syncthreads();
        for (int u = 0; u < nt; ++u) {
            const float xv = sx[u * SCAN_CH + cl], dt = sdt[u * SCAN_CH + cl];
            const float dx = dt * xv;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NPL; ++j) {
                const int n = l + SCAN_LANES * j;
                if (n < N) {
                    S[j] = fmaf(expf(dt * A[j]), S[j], dx * sB[u * N + n]);
                    acc = fmaf(S[j], sC[u * N + n], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (live && l == 0) {
                float y = fmaf(Dc, xv, acc);
                if (p.z != nullptr) y *= ss_silu(sz[u * SCAN_CH + cl]);
                const size_t o = (size_t)(t0 + u) * p.out_stride + c;
                if (p.out_is_bf16) ((bf16*)p.out)[o] = __float2bfloat16_rn(y); else ((float*)p.out)[o] = y;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        if (live && n < N) st[n] = S[j];
    }
}

extern "C" int odin_selective_scan(const void* x, int x_dtype, long long x_stride, const float* dt, long long dt_stride,
                                   const void* dt_bias, const float* B, const float* C, long long bc_stride,
                                   const void* A_log, const void* D, int w_dtype, const void* z, long long z_stride,
                                   float* state, long long state_stride, void* out, int out_dtype, long long out_stride,
                                   const int* seq_start, const int* seq_slots, int n_seqs, int inner, int N, void* stream) {
    if (n_seqs <= 0) return 0;
    if (inner <= 0 || N <= 0 || N > 32 * SCAN_LANES) return ODIN_ERR_UNSUPPORTED;
    ScanParams p;
    p.x = x; p.x_is_bf16 = x_dtype == ODIN_BF16; p.x_stride = x_stride;
    p.dt = dt; p.dt_stride = dt_stride; p.dt_bias = VecRef{dt_bias, w_dtype == ODIN_BF16};
    p.B = B; p.C = C; p.bc_stride = bc_stride;
    p.A_log = VecRef{A_log, w_dtype == ODIN_BF16}; p.D = VecRef{D, w_dtype == ODIN_BF16};
    p.z = z; p.z_stride = z_stride; p.state = state; p.state_stride = state_stride;
    p.out = out; p.out_is_bf16 = out_dtype == ODIN_BF16; p.out_stride = out_stride;
    p.seq_start = seq_start; p.seq_slots = seq_slots; p.inner = inner; p.N = N;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_seqs, (inner + SCAN_CH - 1) / SCAN_CH);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(2 * SCAN_TOK * N + 3 * SCAN_TOK * SCAN_CH) * sizeof(float);
    const dim3 block(SCAN_CH * SCAN_LANES);
    if (N <= 16) odin_launch(selective_scan_kernel<4>, grid, block, smem, s, p);
    else if (N <= 32) odin_launch(selective_scan_kernel<8>, grid, block, smem, s, p);
    else if (N <= 64) odin_launch(selective_scan_kernel<16>, grid, block, smem, s, p);
    else odin_launch(selective_scan_kernel<32>, grid, block, smem, s, p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ skip, gate and grouped norm after a recurrence over heads
// y[t, h, j] = (o[t, h, j] + D[h] x[t, h, j]) * silu(z[t, h, j]); the row is cut into `groups` equal consecutive parts and
// every part is divided by its own root mean square; out = y * w.  One CTA per token; D, z and w are optional.
template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
skip_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ x, size_t x_stride, VecRef D, int P,
                      const TZ* __restrict__ z, size_t z_stride, VecRef w, int groups, float eps, TO* __restrict__ out,
                      int inner) {
    extern __shared__ float row[];   // inner
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < inner; j += blockDim.x) {
        float y = o[(size_t)t * inner + j];
        if (D.p != nullptr) y = fmaf(D.at(j / P), x[(size_t)t * x_stride + j], y);
        if (z != nullptr) y *= ss_silu(to_f32(z[(size_t)t * z_stride + j]));
        row[j] = y;
    }
    const int gsz = inner / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int j = g * gsz + threadIdx.x; j < (g + 1) * gsz; j += blockDim.x) ss += row[j] * row[j];
        ss = block_sum(ss, red);
        ss /= (float)gsz;
        ss += eps;
        const float rs = 1.0f / sqrtf(ss);
        for (int j = g * gsz + threadIdx.x; j < (g + 1) * gsz; j += blockDim.x)
            out[(size_t)t * inner + j] = from_f32<TO>(w.p != nullptr ? w.at(j) * (rs * row[j]) : rs * row[j]);
    }
}

extern "C" int odin_skip_gate_norm(const float* o, const float* x, long long x_stride, const void* D, int P, const void* z,
                                   int z_dtype, long long z_stride, const void* w, int w_dtype, int groups, float eps,
                                   void* out, int out_dtype, int T, int inner, void* stream) {
    if (T <= 0) return 0;
    if (inner <= 0 || groups < 1 || inner % groups != 0 || P <= 0) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)inner * sizeof(float);
    if (smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef Dv{D, w_dtype == ODIN_BF16}, wv{w, w_dtype == ODIN_BF16};
#define GO(TZ, TO)                                                                                                      \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(skip_gate_norm_kernel<TZ, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                        \
        }                                                                                                               \
        odin_launch(skip_gate_norm_kernel<TZ, TO>, dim3(T), dim3(256), smem, s, o, x, (size_t)x_stride, Dv, P, (const TZ*)z, \
                    (size_t)z_stride, wv, groups, eps, (TO*)out, inner);                                                \
    } while (0)
    if (z_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (z_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else if (z_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else if (z_dtype == ODIN_BF16 && out_dtype == ODIN_F32) GO(bf16, float);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}
