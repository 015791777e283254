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
// store: every sequence brings one row (a decode step), and the thread that has read its channel's memory writes the new one
// itself (no other thread touches that channel of that slot); else a second kernel stores the memory.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const TI* __restrict__ in, size_t in_stride, VecRef w, VecRef bias, int taps, int silu,
                   float* __restrict__ state, size_t state_stride, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slots, TO* __restrict__ out,
                   size_t out_stride, int C, int store) {
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
    if (store && taps > 1) {   // t == first: the memory moves up by one row and takes this row's input
        float* st = state + (size_t)slot * state_stride + c;
        for (int k = 0; k + 2 < taps; ++k) st[(size_t)k * C] = st[(size_t)(k + 1) * C];
        st[(size_t)(taps - 2) * C] = to_f32(in[(size_t)t * in_stride + c]);
    }
}

// Up to four taps: a thread takes one channel over CONV_TOK rows in turn, its weights and the last three inputs in
// registers, so that a row costs one load and one store (the window is fetched anew where a sequence's rows begin).
// The same sum in the same order as above (a tap that the filter does not have multiplies nothing and is left out).
#define CONV_TOK 16
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_conv4_kernel(const TI* __restrict__ in, size_t in_stride, VecRef w, VecRef bias, int taps, int silu,
                    const float* __restrict__ state, size_t state_stride, const int* __restrict__ tok_seq,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_slots, TO* __restrict__ out,
                    size_t out_stride, int C, int T) {
    pdl_trigger();
    const int t0 = blockIdx.x * CONV_TOK, t1 = min(T, t0 + CONV_TOK);
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    float wv[4] = {0.f, 0.f, 0.f, 0.f};   // wv[3] meets the current row, wv[3 - m] the row m before
    float b = 0.f;
    if (c < C) {
        for (int j = 0; j < taps; ++j) wv[4 - taps + j] = w.at(c * taps + j);
        if (bias.p != nullptr) b = bias.at(c);
    }
    pdl_wait();
    if (c >= C) return;
    float win[3] = {0.f, 0.f, 0.f};       // win[m - 1]: the input m rows before
    int have = -1;                        // the sequence whose rows the window holds
    for (int t = t0; t < t1; ++t) {
        const int seq = tok_seq[t];
        if (seq < 0) { have = -1; continue; }
        const int first = seq_start[seq];
        if (seq != have || t == first) {
            const int slot = seq_slots[seq];
#pragma unroll
            for (int m = 1; m <= 3; ++m) {
                float v = 0.f;
                if (m < taps) {
                    const int r = t - m;
                    v = r >= first ? to_f32(in[(size_t)r * in_stride + c])
                                   : state[(size_t)slot * state_stride + (size_t)(taps - 1 - (first - r)) * C + c];
                }
                win[m - 1] = v;
            }
            have = seq;
        }
        const float cur = to_f32(in[(size_t)t * in_stride + c]);
        float acc = b;
        if (taps > 3) acc = fmaf(wv[0], win[2], acc);
        if (taps > 2) acc = fmaf(wv[1], win[1], acc);
        if (taps > 1) acc = fmaf(wv[2], win[0], acc);
        acc = fmaf(wv[3], cur, acc);
        out[(size_t)t * out_stride + c] = from_f32<TO>(silu ? ss_silu(acc) : acc);
        win[2] = win[1]; win[1] = win[0]; win[0] = cur;
    }
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
                                int out_dtype, long long out_stride, int T, int C, int single_rows, void* stream) {
    if (T <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > 64 || n_seqs <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef wv{w, w_dtype == ODIN_BF16}, bv{bias, bias_dtype == ODIN_BF16};
    const int threads = C >= 256 ? 256 : (C + 31) / 32 * 32;
    dim3 grid(T, (C + threads - 1) / threads);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
    const dim3 grid4((T + CONV_TOK - 1) / CONV_TOK, grid.y);
#define GO(TI, TO)                                                                                                   \
    do {                                                                                                             \
        if (taps <= 4 && T > 64 && !single_rows)                                                                     \
            odin_launch(causal_conv4_kernel<TI, TO>, grid4, dim3(threads), 0, s, (const TI*)in, (size_t)in_stride, wv, bv, \
                        taps, silu, (const float*)state, (size_t)state_stride, tok_seq, seq_start, seq_slots, (TO*)out, \
                        (size_t)out_stride, C, T);                                                                   \
        else                                                                                                         \
            odin_launch(causal_conv_kernel<TI, TO>, grid, dim3(threads), 0, s, (const TI*)in, (size_t)in_stride, wv, bv, \
                        taps, silu, state, (size_t)state_stride, tok_seq, seq_start, seq_slots, (TO*)out,           \
                        (size_t)out_stride, C, single_rows);                                                         \
    } while (0)
    if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_F32) GO(bf16, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    if (taps > 1 && !single_rows) {
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
    // Blocks of tokens (block_len > 0): a CTA walks one block of one sequence from a state of zeros and leaves the block's
    // own state in s_loc, the sum of its step sizes per channel in dtot, per token the sum since the block's start in cumdt
    // and the output so far (before the gate) in ytmp; a second kernel carries the state from block to block, a third adds
    // what each block's incoming state contributes to its tokens' outputs and applies the gate.
    int block_len, n_blocks;
    float* ytmp;    // [rows, inner]
    float* cumdt;   // [rows, inner]
    float* s_loc;   // [sequences * n_blocks][inner][N]
    float* dtot;    // [sequences * n_blocks][inner]
};

template <int NPL, bool BLOCKS>
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
    const int b = BLOCKS ? blockIdx.x / p.n_blocks : blockIdx.x, ch0 = blockIdx.y * SCAN_CH;
    const int cl = threadIdx.x / SCAN_LANES, l = threadIdx.x % SCAN_LANES;
    const int c = ch0 + cl;
    const bool live = c < p.inner;
    const int seq_end = p.seq_start[b + 1];
    const int row0 = p.seq_start[b] + (BLOCKS ? (int)(blockIdx.x % p.n_blocks) * p.block_len : 0);
    const int row1 = BLOCKS ? min(seq_end, row0 + p.block_len) : seq_end;
    const int slot = p.seq_slots[b];
    float A[NPL], S[NPL];
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        A[j] = (live && n < N) ? -expf(p.A_log.at(c * N + n)) : 0.f;
    }
    const float Dc = (live && p.D.p != nullptr) ? p.D.at(c) : 0.f;
    pdl_wait();
    if (row1 <= row0) return;   // an empty (padding) sequence owns no state
    float* st = BLOCKS ? p.s_loc + ((size_t)blockIdx.x * p.inner + c) * N
                       : p.state + (size_t)slot * p.state_stride + (size_t)c * N;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        S[j] = (!BLOCKS && live && n < N) ? st[n] : 0.f;
    }
    float cum = 0.f;
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
            if (BLOCKS) cum += dt;
            if (live && l == 0) {
                float y = fmaf(Dc, xv, acc);
                if (BLOCKS) {
                    p.ytmp[(size_t)(t0 + u) * p.inner + c] = y;
                    p.cumdt[(size_t)(t0 + u) * p.inner + c] = cum;
                } else {
                    if (p.z != nullptr) y *= ss_silu(sz[u * SCAN_CH + cl]);
                    const size_t o = (size_t)(t0 + u) * p.out_stride + c;
                    if (p.out_is_bf16) ((bf16*)p.out)[o] = __float2bfloat16_rn(y); else ((float*)p.out)[o] = y;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        if (live && n < N) st[n] = S[j];
    }
    if (BLOCKS && live && l == 0) p.dtot[(size_t)blockIdx.x * p.inner + c] = cum;
}

// The state from block to block: S_in(first block) = the sequence's state; S_in(next) = exp(A dtot) S_in + s_loc.
// s_loc is overwritten with S_in (what the block's tokens look at); the last S becomes the sequence's state.
__global__ void __launch_bounds__(256)
scan_carry_kernel(ScanParams p) {
    pdl_trigger();
    const int b = blockIdx.x;
    const int e = blockIdx.y * blockDim.x + threadIdx.x;   // (channel, state index)
    const int row0 = p.seq_start[b], row1 = p.seq_start[b + 1], slot = p.seq_slots[b];
    pdl_wait();
    if (row1 <= row0 || e >= p.inner * p.N) return;
    const int c = e / p.N;
    const float A = -expf(p.A_log.at(e));
    float* st = p.state + (size_t)slot * p.state_stride + e;
    float S = *st;
    const int n = (row1 - row0 + p.block_len - 1) / p.block_len;
    for (int k = 0; k < n; ++k) {
        const size_t item = (size_t)b * p.n_blocks + k;
        const float own = p.s_loc[item * p.inner * p.N + e];
        p.s_loc[item * p.inner * p.N + e] = S;
        S = fmaf(expf(A * p.dtot[item * p.inner + c]), S, own);
    }
    *st = S;
}

// out[t, c] = (ytmp[t, c] + sum_n C_t[n] exp(A[c, n] cumdt[t, c]) S_in[c, n]) * silu(z[t, c]) for the tokens of one block.
template <int NPL>
__global__ void __launch_bounds__(SCAN_CH * SCAN_LANES)
scan_carry_out_kernel(ScanParams p) {
    extern __shared__ float scan_sm[];
    const int N = p.N;
    float* sC = scan_sm;   // [SCAN_TOK][N]
    pdl_trigger();
    const int item = blockIdx.x, b = item / p.n_blocks, ch0 = blockIdx.y * SCAN_CH;
    const int cl = threadIdx.x / SCAN_LANES, l = threadIdx.x % SCAN_LANES;
    const int c = ch0 + cl;
    const bool live = c < p.inner;
    const int seq_end = p.seq_start[b + 1];
    const int row0 = p.seq_start[b] + (item % p.n_blocks) * p.block_len;
    const int row1 = min(seq_end, row0 + p.block_len);
    float A[NPL], Sin[NPL];
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        A[j] = (live && n < N) ? -expf(p.A_log.at(c * N + n)) : 0.f;
    }
    pdl_wait();
    if (row1 <= row0) return;
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = l + SCAN_LANES * j;
        Sin[j] = (live && n < N) ? p.s_loc[((size_t)item * p.inner + c) * N + n] : 0.f;
    }
    float* scd = sC + SCAN_TOK * N;            // [SCAN_TOK][SCAN_CH] sums of steps, outputs so far, gates
    float* sy = scd + SCAN_TOK * SCAN_CH;
    float* sz = sy + SCAN_TOK * SCAN_CH;
    for (int t0 = row0; t0 < row1; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, row1 - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < nt * N; e += blockDim.x) sC[e] = p.C[(size_t)(t0 + e / N) * p.bc_stride + e % N];
        for (int e = threadIdx.x; e < nt * SCAN_CH; e += blockDim.x) {
            const int cc = ch0 + e % SCAN_CH;
            const size_t r = (size_t)(t0 + e / SCAN_CH);
            float cd = 0.f, yv = 0.f, zv = 0.f;
            if (cc < p.inner) {
                cd = p.cumdt[r * p.inner + cc];
                yv = p.ytmp[r * p.inner + cc];
                if (p.z != nullptr)
                    zv = p.x_is_bf16 ? __bfloat162float(((const bf16*)p.z)[r * p.z_stride + cc]) : ((const float*)p.z)[r * p.z_stride + cc];
            }
            scd[e] = cd; sy[e] = yv; sz[e] = zv;
        }
        __syncthreads();
        for (int u = 0; u < nt; ++u) {
            const float cd = scd[u * SCAN_CH + cl];
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NPL; ++j) {
                const int n = l + SCAN_LANES * j;
                if (n < N) acc = fmaf(expf(cd * A[j]) * Sin[j], sC[u * N + n], acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (live && l == 0) {
                float y = sy[u * SCAN_CH + cl] + acc;
                if (p.z != nullptr) y *= ss_silu(sz[u * SCAN_CH + cl]);
                const size_t o = (size_t)(t0 + u) * p.out_stride + c;
                if (p.out_is_bf16) ((bf16*)p.out)[o] = __float2bfloat16_rn(y); else ((float*)p.out)[o] = y;
            }
        }
    }
}

extern "C" int odin_selective_scan(const void* x, int x_dtype, long long x_stride, const float* dt, long long dt_stride,
                                   const void* dt_bias, const float* B, const float* C, long long bc_stride,
                                   const void* A_log, const void* D, int w_dtype, const void* z, long long z_stride,
                                   float* state, long long state_stride, void* out, int out_dtype, long long out_stride,
                                   const int* seq_start, const int* seq_slots, int n_seqs, int inner, int N, int block_len,
                                   int n_blocks, float* ytmp, float* cumdt, float* s_loc, float* dtot, void* stream) {
    if (n_seqs <= 0) return 0;
    if (inner <= 0 || N <= 0 || N > 64 * SCAN_LANES) return ODIN_ERR_UNSUPPORTED;
    if (block_len < 0 || (block_len > 0 && (n_blocks <= 0 || ytmp == nullptr || cumdt == nullptr || s_loc == nullptr ||
                                            dtot == nullptr || (long long)n_seqs * n_blocks > 2147483647LL)))
        return ODIN_ERR_BAD_ARG;
    ScanParams p;
    p.x = x; p.x_is_bf16 = x_dtype == ODIN_BF16; p.x_stride = x_stride;
    p.dt = dt; p.dt_stride = dt_stride; p.dt_bias = VecRef{dt_bias, w_dtype == ODIN_BF16};
    p.B = B; p.C = C; p.bc_stride = bc_stride;
    p.A_log = VecRef{A_log, w_dtype == ODIN_BF16}; p.D = VecRef{D, w_dtype == ODIN_BF16};
    p.z = z; p.z_stride = z_stride; p.state = state; p.state_stride = state_stride;
    p.out = out; p.out_is_bf16 = out_dtype == ODIN_BF16; p.out_stride = out_stride;
    p.seq_start = seq_start; p.seq_slots = seq_slots; p.inner = inner; p.N = N;
    p.block_len = block_len; p.n_blocks = n_blocks; p.ytmp = ytmp; p.cumdt = cumdt; p.s_loc = s_loc; p.dtot = dtot;
    cudaStream_t s = (cudaStream_t)stream;
    const bool blocks = block_len > 0;
    dim3 grid(blocks ? n_seqs * n_blocks : n_seqs, (inner + SCAN_CH - 1) / SCAN_CH);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(2 * SCAN_TOK * N + 3 * SCAN_TOK * SCAN_CH) * sizeof(float);
    const dim3 block(SCAN_CH * SCAN_LANES);
#define GO(NPL)                                                                                     \
    do {                                                                                            \
        if (blocks) odin_launch(selective_scan_kernel<NPL, true>, grid, block, smem, s, p);         \
        else odin_launch(selective_scan_kernel<NPL, false>, grid, block, smem, s, p);               \
    } while (0)
    if (N <= 16) GO(4);
    else if (N <= 32) GO(8);
    else if (N <= 64) GO(16);
    else if (N <= 128) GO(32);
    else GO(64);
#undef GO
    ODIN_LAUNCH_CHECK();
    if (blocks) {
        odin_launch(scan_carry_kernel, dim3(n_seqs, (inner * N + 255) / 256), dim3(256), 0, s, p);
        ODIN_LAUNCH_CHECK();
        const size_t sm2 = (size_t)(SCAN_TOK * N + 3 * SCAN_TOK * SCAN_CH) * sizeof(float);
        if (N <= 16) odin_launch(scan_carry_out_kernel<4>, grid, block, sm2, s, p);
        else if (N <= 32) odin_launch(scan_carry_out_kernel<8>, grid, block, sm2, s, p);
        else if (N <= 64) odin_launch(scan_carry_out_kernel<16>, grid, block, sm2, s, p);
        else if (N <= 128) odin_launch(scan_carry_out_kernel<32>, grid, block, sm2, s, p);
        else odin_launch(scan_carry_out_kernel<64>, grid, block, sm2, s, p);
        ODIN_LAUNCH_CHECK();
    }
    return 0;
}

// ------------------------------------------------------------ skip, gate and grouped norm after a recurrence over heads
// y[t, h, j] = (o[t, h, j] + D[h] x[t, h, j]) * silu(z[t, h, j]); the row is cut into `groups` equal consecutive parts and
// every part is divided by its own root mean square; out = y * w.  One CTA per (token, part); D, z and w are optional.
template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
skip_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ x, size_t x_stride, VecRef D, int P,
                      const TZ* __restrict__ z, size_t z_stride, VecRef w, int groups, float eps, TO* __restrict__ out,
                      int inner) {
    extern __shared__ float row[];   // one part of the row
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y;
    const int gsz = inner / groups, j0 = g * gsz;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gsz; i += blockDim.x) {
        const int j = j0 + i;
        float y = o[(size_t)t * inner + j];
        if (D.p != nullptr) y = fmaf(D.at(j / P), x[(size_t)t * x_stride + j], y);
        if (z != nullptr) y *= ss_silu(to_f32(z[(size_t)t * z_stride + j]));
        row[i] = y;
        ss += y * y;
    }
    ss = block_sum(ss, red);
    ss /= (float)gsz;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    for (int i = threadIdx.x; i < gsz; i += blockDim.x)
        out[(size_t)t * inner + j0 + i] = from_f32<TO>(w.p != nullptr ? w.at(j0 + i) * (rs * row[i]) : rs * row[i]);
}

extern "C" int odin_skip_gate_norm(const float* o, const float* x, long long x_stride, const void* D, int P, const void* z,
                                   int z_dtype, long long z_stride, const void* w, int w_dtype, int groups, float eps,
                                   void* out, int out_dtype, int T, int inner, void* stream) {
    if (T <= 0) return 0;
    if (inner <= 0 || groups < 1 || inner % groups != 0 || P <= 0) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)(inner / groups) * sizeof(float);
    if (smem > 200 * 1024 || groups > 65535) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef Dv{D, w_dtype == ODIN_BF16}, wv{w, w_dtype == ODIN_BF16};
    const int threads = inner / groups >= 1024 ? 256 : 128;
#define GO(TZ, TO)                                                                                                      \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(skip_gate_norm_kernel<TZ, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                        \
        }                                                                                                               \
        odin_launch(skip_gate_norm_kernel<TZ, TO>, dim3(T, groups), dim3(threads), smem, s, o, x, (size_t)x_stride, Dv, P, (const TZ*)z, \
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
