// Mixers that keep a fixed-size state per sequence instead of keys and values:
//
//   * token shift: every stream s of a mixer reads h_t + (h_(t-1) - h_t) * mu_s, where h_(t-1)
//     is the row before in the same sequence or, for a step's first token, the row that the
//     sequence's state holds (zeros at the start of a sequence);
//   * the linear recurrence over a matrix-valued state S (key channel x value channel) per head,
//         o_t = (diag(a_t) S_(t-1) + diag(b) k_t v_t^T)^T q_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T,
//     in its two uses: with a = 1 and a bonus b = u for the current token (output before the
//     decay: the "wkv" form), and with a = w, b = 1 (output after the update: the gated form in
//     which the forget gate f also scales what is written, k = 1 - f); and with a = w = one constant per head
//     (retention: no gate, the keys and queries as they come, output after the update);
//   * the per-head unit norm of the recurrence's output, times a weight, times an optional gate.
//
// The state lives in 32-bit floats in the engine's per-sequence state area and is carried from
// step to step; a sequence's tokens are walked in order by one CTA per (sequence, head), column j of S
// held in the registers of four lanes, so the result does not depend on how the tokens were cut into
// steps or on what else is in the batch.  Decays, gates, exponentials and the state are 32-bit.
#include "common.cuh"

// ------------------------------------------------------------ token shift
// out[s][t][:] = h[t] + (prev - h[t]) * mu[s], s < n_mix.  Rows of sequence -1 are skipped.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state, size_t state_stride, VecRef mu, int n_mix,
                   T* __restrict__ out, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                   const int* __restrict__ seq_slots, int n_rows, int d) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int seq = tok_seq[t];
    int first = 0, slot = 0;
    if (seq >= 0) { first = seq_start[seq]; slot = seq_slots[seq]; }
    pdl_wait();
    if (seq < 0) return;
    const T* hr = h + (size_t)t * d;
    if (VEC) {  // the width a multiple of four, every row 16-byte aligned
        for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
            const float4 hv = ld4(hr + c);
            const float4 pv = (t == first) ? ld4(state + (size_t)slot * state_stride + c) : ld4(hr + c - d);
            const float4 diff = make_float4(pv.x - hv.x, pv.y - hv.y, pv.z - hv.z, pv.w - hv.w);
            for (int s = 0; s < n_mix; ++s) {
                const float4 m = mu.at4(s * d + c);
                st4(out + ((size_t)s * n_rows + t) * d + c,
                    make_float4(hv.x + diff.x * m.x, hv.y + diff.y * m.y, hv.z + diff.z * m.z, hv.w + diff.w * m.w));
            }
        }
    }
    for (int c = threadIdx.x; !VEC && c < d; c += blockDim.x) {
        const float hv = to_f32(hr[c]);
        const float pv = (t == first) ? state[(size_t)slot * state_stride + c] : to_f32(hr[c - d]);
        const float diff = pv - hv;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * n_rows + t) * d + c] = from_f32<T>(hv + diff * mu.at(s * d + c));
    }
}

extern "C" int odin_token_shift(const void* h, int dtype, const float* state, long long state_stride, const void* mu,
                                int mu_dtype, int n_mix, void* out, const int* tok_seq, const int* seq_start,
                                const int* seq_slots, int n_rows, int d, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0 || n_mix <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef mv{mu, mu_dtype == ODIN_BF16};
    const bool vec = (d % 4 == 0) && (state_stride % 4 == 0) &&
                     ((((uintptr_t)h) | ((uintptr_t)state) | ((uintptr_t)mu) | ((uintptr_t)out)) % 16 == 0);
    if (dtype == ODIN_BF16)
        odin_launch(vec ? token_shift_kernel<bf16, true> : token_shift_kernel<bf16, false>, dim3(n_rows), dim3(256), 0, s,
                    (const bf16*)h, state, (size_t)state_stride, mv, n_mix, (bf16*)out, tok_seq, seq_start, seq_slots, n_rows, d);
    else if (dtype == ODIN_F32)
        odin_launch(vec ? token_shift_kernel<float, true> : token_shift_kernel<float, false>, dim3(n_rows), dim3(256), 0, s,
                    (const float*)h, state, (size_t)state_stride, mv, n_mix, (float*)out, tok_seq, seq_start, seq_slots, n_rows, d);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ the recurrence
#define REC_BONUS 0   // o = (S + diag(u) k v^T)^T r, then S = diag(w) S + k v^T, w = exp(-exp(raw + w0))
#define REC_GATED 1   // f = l + (1 - l) sigmoid(raw + b); S = diag(f) S + (1 - f) v^T; o = S^T silu(q)
#define REC_FIXED 2   // S = c0 S + k v^T; o = S^T q: a decay that is one constant per head (c0: [H])
#define REC_GLA 3     // w = sigmoid(raw + c0)^c1 = exp(c1 logsigmoid(raw + c0)); S = diag(w) S + k v^T; o = S^T (q_scale q)
#define REC_SSD 4     // per head and token one step dt = softplus(raw[head] + c1[head]) and one decay w = exp(-exp(c0[head]) dt);
                      // S = w S + (dt k) v^T; o = S^T q; q and k belong to the head's group (heads_per_group heads share them)
// Threads that share a column of S: each owns a quarter of the key channels.  (Sixteen lanes per column, a quarter of
// the registers each, walked a prompt of 2,048 tokens a fifth faster and made a decode step three to four times slower:
// four times the threads for the same work.)
#define REC_SPLIT 4
#define REC_MAX_DK 256

struct RecParams {
    const float* q; long long q_stride;   // [rows, H*dk] projections (32-bit), row strides in elements
    const float* k; long long k_stride;   // REC_BONUS and REC_FIXED
    const float* g; long long g_stride;   // the raw decay / forget gate (REC_FIXED: unused)
    const float* v; long long v_stride;   // [rows, H*dv]
    VecRef c0, c1;                        // per (head, key channel): REC_BONUS w0 and u; REC_GATED bias and lower bound; REC_FIXED: c0 per head
    float* o; long long o_stride;         // [rows, H*dv]
    float* state; long long state_stride; // per slot: [H][dk][dv] floats
    const int* seq_start; const int* seq_slots;
    int H, dk, dv;
    float q_scale;        // REC_GLA: factor on q
    int heads_per_group;  // REC_SSD: heads that share one q and one k (their columns: group * dk)
    // the token shift's memory: after the step the sequence's last row of h goes to its state
    const void* shift_src; int shift_is_bf16; float* shift_state; long long shift_stride; int width;
    // Blocks of tokens (block_len > 0): a CTA walks one block of one sequence from a state of zeros and leaves
    // the block's own state in s_loc, the product of the block's decays per key channel in d_tot, and per token
    // q times the decays since the block's start in qp; two small kernels then carry the state from block to block
    // and add what each block's incoming state contributes to its tokens' outputs.
    int block_len, n_blocks;
    float* qp;     // [rows, H*dk]
    float* s_loc;  // [sequences * n_blocks][H][dk][dv]
    float* d_tot;  // [sequences * n_blocks][H*dk]
};

// One CTA per (sequence, head) walks the sequence's tokens in order.  Column j of S belongs to REC_SPLIT lanes of
// one warp (lane = part * 8 + j % 8), each holding SL consecutive key channels of it in registers; a token costs
// each thread SL multiply-adds for the output and SL for the state, and the column's output is the sum of its
// parts' shares (two shuffles), always added in the same order.  The tokens' q, k, decays and values are prepared a
// block of tokens at a time in shared memory (the exponentials once per token and channel, not once per column);
// the next block's inputs are fetched into registers before the current block is walked, so that the walk itself
// reads shared memory only.
// A CTA covers `cols` columns (a multiple of 8, at most REC_COLS; blockIdx.z takes the next ones), so that it never
// has more than 512 threads and the state fits the registers; the launcher takes fewer columns per CTA when there
// are few (sequence, head) pairs, so that a long prompt of one sequence still occupies the GPU.  A column's
// arithmetic does not depend on which CTA holds it.
#define REC_COLS 128
#define REC_FETCH 4   // elements of each input that a thread fetches ahead per block of tokens
template <int SL, int MODE, bool BLOCKS>
__global__ void __launch_bounds__(REC_COLS * REC_SPLIT)
linear_recurrence_kernel(RecParams p) {
    constexpr int NK = SL * REC_SPLIT;             // key channels the registers hold (dk <= NK)
    constexpr int TOK = NK > 128 ? 8 : 16;
    constexpr bool BONUS_IN_REGS = SL <= 32;
    constexpr bool UNI = MODE == REC_FIXED || MODE == REC_SSD;   // one decay for the whole head: a register, no row of shared memory
    __shared__ float s_wt[TOK], s_dt[TOK];         // REC_SSD: the token's decay and step, formed once per token
    // A warp's four parts read their channels at the same moment, SL floats apart: every part's channels sit four floats
    // further on than the part before, so that the four 16-byte reads fall into different banks (SL = 32: banks 0, 4, 8, 12
    // in place of four times bank 0).
    constexpr int NKP = NK + 4 * REC_SPLIT;
    __shared__ __align__(16) float sq[TOK][NKP], sk[TOK][NKP], sw[TOK][NKP];
    __shared__ float sv[TOK][REC_COLS], sb[NK];
    pdl_trigger();
    const int b = BLOCKS ? blockIdx.x / p.n_blocks : blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ccols = blockDim.x / REC_SPLIT;      // columns of this CTA
    const int part = lane >> 3, cj = warp * 8 + (lane & 7), j = blockIdx.z * ccols + cj;
    const int dk = p.dk;
    const int seq_end = p.seq_start[b + 1];
    const int row0 = p.seq_start[b] + (BLOCKS ? (int)(blockIdx.x % p.n_blocks) * p.block_len : 0);
    const int row1 = BLOCKS ? min(seq_end, row0 + p.block_len) : seq_end;
    const int slot = p.seq_slots[b];
    const int hc = head * dk;
    const int qc = MODE == REC_SSD ? (head / p.heads_per_group) * dk : hc;   // the head's columns of q and k
    const int tok = max(1, min(TOK, REC_FETCH * (int)blockDim.x / NK));   // tokens per block: what the threads can fetch ahead
    for (int i = threadIdx.x; i < NK; i += blockDim.x) sb[i] = (MODE == REC_BONUS && i < dk) ? p.c1.at(hc + i) : 0.f;
    pdl_wait();
    if (row1 <= row0) return;  // an empty (padding) sequence owns no state
    const bool owns = j < p.dv;
    const int i0 = part * SL;
    float S[SL], ub[BONUS_IN_REGS ? SL : 1], D[(BLOCKS && !UNI) ? SL : 1];
    const float wuni = MODE == REC_FIXED ? p.c0.at(head) : 0.f;
    float* st = BLOCKS ? p.s_loc + ((size_t)blockIdx.x * p.H + head) * dk * p.dv + j
                       : p.state + (size_t)slot * p.state_stride + (size_t)head * dk * p.dv + j;
#pragma unroll
    for (int i = 0; i < SL; ++i) S[i] = (!BLOCKS && owns && i0 + i < dk) ? st[(size_t)(i0 + i) * p.dv] : 0.f;
    if (BLOCKS) {
#pragma unroll
        for (int i = 0; i < (UNI ? 1 : SL); ++i) D[i] = 1.0f;
    }
    const bool writes_qp = BLOCKS && cj == 0 && blockIdx.z == 0;   // one column's lanes write what is per key channel
    __syncthreads();
    if (BONUS_IN_REGS) {
#pragma unroll
        for (int i = 0; i < SL; ++i) ub[i] = sb[i0 + i];
    }

    float rq[REC_FETCH], rk[REC_FETCH], rg[REC_FETCH], rv[REC_FETCH];
    auto fetch = [&](int t0, int nt) {
#pragma unroll
        for (int f = 0; f < REC_FETCH; ++f) {
            const int e = threadIdx.x + f * blockDim.x;
            rq[f] = rk[f] = rg[f] = rv[f] = 0.f;
            if (e < nt * NK) {
                const int u = e / NK, i = e % NK;
                if (i < dk) {
                    const size_t r = (size_t)(t0 + u);
                    rq[f] = p.q[r * p.q_stride + qc + i];
                    if (MODE == REC_SSD) rg[f] = p.g[r * p.g_stride + head];
                    else if (MODE != REC_FIXED) rg[f] = p.g[r * p.g_stride + hc + i];
                    if (MODE != REC_GATED) rk[f] = p.k[r * p.k_stride + qc + i];
                }
            }
            if (e < nt * ccols) {
                const int u = e / ccols, c = e % ccols, col = blockIdx.z * ccols + c;
                if (col < p.dv) rv[f] = p.v[(size_t)(t0 + u) * p.v_stride + (size_t)head * p.dv + col];
            }
        }
    };
    auto commit = [&](int nt) {
#pragma unroll
        for (int f = 0; f < REC_FETCH; ++f) {
            const int e = threadIdx.x + f * blockDim.x;
            if (e < nt * NK) {
                const int u = e / NK, i = e % NK;
                float qv = 0.f, kv = 0.f, wv = 0.f;   // channels beyond dk: nothing in, nothing kept
                if (i < dk) {
                    if (MODE == REC_BONUS) {
                        qv = rq[f];
                        kv = rk[f];
                        wv = expf(-expf(rg[f] + p.c0.at(hc + i)));
                    } else if (MODE == REC_FIXED) {
                        qv = rq[f];
                        kv = rk[f];
                    } else if (MODE == REC_GLA) {
                        const float z = rg[f] + p.c0.at(hc + i);
                        const float logsig = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
                        qv = rq[f] * p.q_scale;
                        kv = rk[f];
                        wv = expf(p.c1.at(hc + i) * logsig);
                    } else if (MODE == REC_SSD) {
                        qv = rq[f];
                        kv = rk[f];       // the step multiplies the token's values once instead of every key channel
                        if (i == 0) {
                            const float z = rg[f] + p.c1.at(head);
                            const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
                            s_dt[u] = dt;
                            s_wt[u] = expf(-expf(p.c0.at(head)) * dt);
                        }
                    } else {
                        const float l = p.c1.at(hc + i);
                        const float fg = l + (1.0f - l) * (1.0f / (1.0f + expf(-(rg[f] + p.c0.at(hc + i)))));
                        qv = rq[f] / (1.0f + expf(-rq[f]));
                        kv = 1.0f - fg;
                        wv = fg;
                    }
                }
                const int ip = i + (i / SL) * 4;
                sq[u][ip] = qv; sk[u][ip] = kv;
                if (!UNI) sw[u][ip] = wv;
            }
            if (e < nt * ccols) sv[e / ccols][e % ccols] = rv[f];
        }
    };

    fetch(row0, min(tok, row1 - row0));
    for (int t0 = row0; t0 < row1; t0 += tok) {
        const int nt = min(tok, row1 - t0);
        __syncthreads();   // the block before has been walked
        commit(nt);
        __syncthreads();
        if (t0 + tok < row1) fetch(t0 + tok, min(tok, row1 - t0 - tok));
        for (int u = 0; u < nt; ++u) {
            const float vj = MODE == REC_SSD ? sv[u][cj] * s_dt[u] : sv[u][cj];
            const float wt = MODE == REC_SSD ? s_wt[u] : wuni;
            float acc0 = 0.f, acc1 = 0.f;
            if (BLOCKS && UNI) D[0] *= wt;   // the output looks at the state after the token's own decay
#pragma unroll
            for (int i4 = 0; i4 < SL; i4 += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[u][i0 + part * 4 + i4]);
                const float4 q4 = *reinterpret_cast<const float4*>(&sq[u][i0 + part * 4 + i4]);
                float4 w4 = make_float4(wt, wt, wt, wt);
                if (!UNI) w4 = *reinterpret_cast<const float4*>(&sw[u][i0 + part * 4 + i4]);
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = i4 + e;
                    const float kv = kk[e] * vj;
                    if (BLOCKS) {
                        // q times the decays between the block's start and this token's look at the state:
                        // before its own decay where the output comes before the update, after it else
                        constexpr int di = (BLOCKS && !UNI) ? 1 : 0;   // D[i * di]: the channel's own product, or the head's one
                        if (MODE != REC_BONUS && !UNI) D[i * di] *= ww[e];
                        if (writes_qp && i0 + i < dk)
                            p.qp[(size_t)(t0 + u) * p.H * dk + hc + i0 + i] = qq[e] * D[i * di];
                        if (MODE == REC_BONUS) D[i * di] *= ww[e];
                    }
                    if (MODE == REC_BONUS) {
                        const float bonus = BONUS_IN_REGS ? ub[BONUS_IN_REGS ? i : 0] : sb[i0 + i];
                        const float term = qq[e] * fmaf(bonus, kv, S[i]);
                        if (e & 1) acc1 += term; else acc0 += term;
                        S[i] = fmaf(ww[e], S[i], kv);
                    } else {
                        S[i] = fmaf(ww[e], S[i], kv);
                        if (e & 1) acc1 = fmaf(qq[e], S[i], acc1); else acc0 = fmaf(qq[e], S[i], acc0);
                    }
                }
            }
            float acc = acc0 + acc1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (owns && part == 0) p.o[(size_t)(t0 + u) * p.o_stride + (size_t)head * p.dv + j] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < SL; ++i)
        if (owns && i0 + i < dk) st[(size_t)(i0 + i) * p.dv] = S[i];
    if (writes_qp) {
#pragma unroll
        for (int i = 0; i < SL; ++i)
            if (i0 + i < dk) p.d_tot[(size_t)blockIdx.x * p.H * dk + hc + i0 + i] = D[(BLOCKS && !UNI) ? i : 0];
    }
    if (head == 0 && blockIdx.z == 0 && p.shift_src != nullptr && row1 == seq_end) {
        float* dst = p.shift_state + (size_t)slot * p.shift_stride;
        const size_t last = (size_t)(row1 - 1) * p.width;
        for (int c = threadIdx.x; c < p.width; c += blockDim.x)
            dst[c] = p.shift_is_bf16 ? __bfloat162float(((const bf16*)p.shift_src)[last + c]) : ((const float*)p.shift_src)[last + c];
    }
}

// The state from block to block: S_in(first block) = the sequence's state; S_in(next) = diag(d_tot) S_in + s_loc.
// s_loc is overwritten with S_in (what the block's tokens look at); the last S becomes the sequence's state.
__global__ void __launch_bounds__(256)
recurrence_carry_kernel(RecParams p) {
    pdl_trigger();
    const int b = blockIdx.x, head = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;   // element of the head's state
    const int row0 = p.seq_start[b], row1 = p.seq_start[b + 1];
    const int slot = p.seq_slots[b];
    pdl_wait();
    if (row1 <= row0 || e >= p.dk * p.dv) return;
    const int i = e / p.dv;
    float* st = p.state + (size_t)slot * p.state_stride + (size_t)head * p.dk * p.dv + e;
    float S = *st;
    const int n = (row1 - row0 + p.block_len - 1) / p.block_len;
    // eight blocks at a time: their loads go out together, then the chain of multiply-adds runs over what came back
    constexpr int CB = 8;
    const size_t per_item = (size_t)p.H * p.dk * p.dv, at = (size_t)head * p.dk * p.dv + e;
    for (int c0 = 0; c0 < n; c0 += CB) {
        const size_t item0 = (size_t)b * p.n_blocks + c0;
        float own[CB], dec[CB];
#pragma unroll
        for (int u = 0; u < CB; ++u) {
            own[u] = dec[u] = 0.f;
            if (c0 + u < n) {
                own[u] = p.s_loc[(item0 + u) * per_item + at];
                dec[u] = p.d_tot[((item0 + u) * p.H + head) * p.dk + i];
            }
        }
#pragma unroll
        for (int u = 0; u < CB; ++u)
            if (c0 + u < n) {
                p.s_loc[(item0 + u) * per_item + at] = S;
                S = fmaf(dec[u], S, own[u]);
            }
    }
    *st = S;
}

// o[t, head, :] += (q_t * decays since the block's start)^T S_in(block): 64 (or 32) tokens by 32 columns per CTA pass.
// Shared memory: the incoming state's 32 columns [dk][32], then (dk a multiple of four) 64 tokens' q [64][dk], which the
// CTA fetches with loads that all go out together; a warp then takes eight tokens and reads four channels of a token's q
// in one broadcast.  Every sum runs over the channels in their order, whichever path computes it.
#define CARRY_OUT_TOK 64
__global__ void __launch_bounds__(256)
recurrence_carry_out_kernel(RecParams p) {
    extern __shared__ __align__(16) float co_smem[];
    float (*tile)[32] = reinterpret_cast<float (*)[32]>(co_smem);
    float* qsm = co_smem + (size_t)p.dk * 32;
    pdl_trigger();
    const int item = blockIdx.x, head = blockIdx.y;
    const int b = item / p.n_blocks;
    const int lane = threadIdx.x & 31, lane_t = threadIdx.x >> 5;
    const int col = blockIdx.z * 32 + lane;
    const int seq_end = p.seq_start[b + 1];
    const int row0 = p.seq_start[b] + (item % p.n_blocks) * p.block_len;
    const int row1 = min(seq_end, row0 + p.block_len);
    pdl_wait();
    if (row1 <= row0) return;
    const float* sin = p.s_loc + ((size_t)item * p.H + head) * p.dk * p.dv;
    for (int e = threadIdx.x; e < p.dk * 32; e += blockDim.x) {
        const int i = e >> 5, c = blockIdx.z * 32 + (e & 31);
        tile[i][e & 31] = c < p.dv ? sin[(size_t)i * p.dv + c] : 0.f;
    }
    const size_t qs = (size_t)p.H * p.dk;
    if ((p.dk & 3) == 0) {
        const int dk4 = p.dk >> 2;
        for (int tb = row0; tb < row1; tb += CARRY_OUT_TOK) {
            __syncthreads();   // the pass before has read its q (and, the first time, the tile is there after the next one)
            for (int e = threadIdx.x; e < CARRY_OUT_TOK * dk4; e += blockDim.x) {
                const int u = e / dk4, c4 = e % dk4;
                if (tb + u < row1)
                    reinterpret_cast<float4*>(qsm)[e] =
                        __ldg(reinterpret_cast<const float4*>(p.qp + (size_t)(tb + u) * qs + (size_t)head * p.dk) + c4);
            }
            __syncthreads();
            const int t0 = tb + lane_t * 8;
            const int nt = min(8, row1 - t0);
            if (nt <= 0) continue;
            float acc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] = 0.f;
            const float* qw = qsm + (size_t)lane_t * 8 * p.dk;
            for (int i = 0; i < p.dk; i += 4) {
                const float s0 = tile[i][lane], s1 = tile[i + 1][lane], s2 = tile[i + 2][lane], s3 = tile[i + 3][lane];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (u < nt) {
                        const float4 q4 = *reinterpret_cast<const float4*>(qw + u * p.dk + i);
                        acc[u] = fmaf(q4.x, s0, acc[u]);
                        acc[u] = fmaf(q4.y, s1, acc[u]);
                        acc[u] = fmaf(q4.z, s2, acc[u]);
                        acc[u] = fmaf(q4.w, s3, acc[u]);
                    }
            }
            if (col < p.dv) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (u < nt) p.o[(size_t)(t0 + u) * p.o_stride + (size_t)head * p.dv + col] += acc[u];
            }
        }
        return;
    }
    __syncthreads();
    for (int t0 = row0 + lane_t * 4; t0 < row1; t0 += 32) {   // a warp takes four tokens at a time
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float* qrow = p.qp + (size_t)t0 * qs + (size_t)head * p.dk;
        for (int i = 0; i < p.dk; ++i) {
            const float sv = tile[i][lane];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (t0 + u < row1) acc[u] = fmaf(__ldg(qrow + u * qs + i), sv, acc[u]);
        }
        if (col < p.dv) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (t0 + u < row1) p.o[(size_t)(t0 + u) * p.o_stride + (size_t)head * p.dv + col] += acc[u];
        }
    }
}

extern "C" int odin_linear_recurrence(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                                      const float* g, long long g_stride, const float* v, long long v_stride,
                                      const void* c0, const void* c1, int c_dtype, float* o, long long o_stride,
                                      float* state, long long state_stride, const int* seq_start, const int* seq_slots,
                                      int n_seqs, int H, int dk, int dv, const void* shift_src, int shift_dtype,
                                      float* shift_state, long long shift_stride, int width, int block_len, int n_blocks,
                                      float* qp, float* s_loc, float* d_tot, float q_scale, int heads_per_group,
                                      void* stream) {
    if (n_seqs <= 0) return 0;
    if (block_len < 0 || (block_len > 0 && (n_blocks <= 0 || qp == nullptr || s_loc == nullptr || d_tot == nullptr ||
                                            (long long)n_seqs * n_blocks > 2147483647LL)))
        return ODIN_ERR_BAD_ARG;
    if (H <= 0 || dk <= 0 || dk > REC_MAX_DK || dv <= 0 || dv > 256 || H > 65535) return ODIN_ERR_UNSUPPORTED;
    if (mode < REC_BONUS || mode > REC_SSD) return ODIN_ERR_BAD_ARG;
    if (mode == REC_SSD && (heads_per_group <= 0 || H % heads_per_group != 0)) return ODIN_ERR_BAD_ARG;
    RecParams p;
    p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.g = g; p.g_stride = g_stride;
    p.v = v; p.v_stride = v_stride;
    p.c0 = VecRef{c0, c_dtype == ODIN_BF16}; p.c1 = VecRef{c1, c_dtype == ODIN_BF16};
    p.o = o; p.o_stride = o_stride; p.state = state; p.state_stride = state_stride;
    p.seq_start = seq_start; p.seq_slots = seq_slots; p.H = H; p.dk = dk; p.dv = dv;
    p.shift_src = shift_src; p.shift_is_bf16 = shift_dtype == ODIN_BF16; p.shift_state = shift_state;
    p.shift_stride = shift_stride; p.width = width;
    p.block_len = block_len; p.n_blocks = n_blocks; p.qp = qp; p.s_loc = s_loc; p.d_tot = d_tot;
    p.q_scale = q_scale; p.heads_per_group = heads_per_group > 0 ? heads_per_group : 1;
    const bool blocks = block_len > 0;
    const int n_items = blocks ? n_seqs * n_blocks : n_seqs;
    cudaStream_t s = (cudaStream_t)stream;
    // columns per CTA: all of them (up to REC_COLS) when (sequence, head) pairs alone fill the GPU twice, else
    // halved down to 32 until they do
    int cols = (dv < REC_COLS ? dv : REC_COLS);
    cols = (cols + 7) / 8 * 8;
    while (cols > 32 && (cols / 2) % 8 == 0 && (long long)n_items * H * ((dv + cols - 1) / cols) < 2 * 148) cols /= 2;
    // a block of tokens is staged by the CTA's threads, REC_FETCH elements each: enough threads for one token's channels
    const int sl = dk <= 16 ? 4 : dk <= 32 ? 8 : dk <= 48 ? 12 : dk <= 64 ? 16 : dk <= 96 ? 24 : dk <= 128 ? 32 : 64;
    if (cols * REC_SPLIT * REC_FETCH < sl * REC_SPLIT) cols = (sl / REC_FETCH + 7) / 8 * 8;
    const int threads = cols * REC_SPLIT;      // a warp per eight columns
    dim3 grid(n_items, H, (dv + cols - 1) / cols);
#define GO(SL)                                                                                                  \
    do {                                                                                                        \
        if (mode == REC_BONUS && blocks) odin_launch(linear_recurrence_kernel<SL, REC_BONUS, true>, grid, dim3(threads), 0, s, p);  \
        else if (mode == REC_BONUS) odin_launch(linear_recurrence_kernel<SL, REC_BONUS, false>, grid, dim3(threads), 0, s, p);     \
        else if (mode == REC_FIXED && blocks) odin_launch(linear_recurrence_kernel<SL, REC_FIXED, true>, grid, dim3(threads), 0, s, p);  \
        else if (mode == REC_FIXED) odin_launch(linear_recurrence_kernel<SL, REC_FIXED, false>, grid, dim3(threads), 0, s, p);     \
        else if (mode == REC_GLA && blocks) odin_launch(linear_recurrence_kernel<SL, REC_GLA, true>, grid, dim3(threads), 0, s, p);  \
        else if (mode == REC_GLA) odin_launch(linear_recurrence_kernel<SL, REC_GLA, false>, grid, dim3(threads), 0, s, p);     \
        else if (mode == REC_SSD && blocks) odin_launch(linear_recurrence_kernel<SL, REC_SSD, true>, grid, dim3(threads), 0, s, p);  \
        else if (mode == REC_SSD) odin_launch(linear_recurrence_kernel<SL, REC_SSD, false>, grid, dim3(threads), 0, s, p);     \
        else if (blocks) odin_launch(linear_recurrence_kernel<SL, REC_GATED, true>, grid, dim3(threads), 0, s, p);  \
        else odin_launch(linear_recurrence_kernel<SL, REC_GATED, false>, grid, dim3(threads), 0, s, p);         \
    } while (0)
    // registers for the smallest multiple of REC_SPLIT channels that holds dk
    if (dk <= 16) GO(4);
    else if (dk <= 32) GO(8);
    else if (dk <= 48) GO(12);
    else if (dk <= 64) GO(16);
    else if (dk <= 96) GO(24);
    else if (dk <= 128) GO(32);
    else GO(64);
#undef GO
    ODIN_LAUNCH_CHECK();
    if (blocks) {
        odin_launch(recurrence_carry_kernel, dim3(n_seqs, H, (dk * dv + 255) / 256), dim3(256), 0, s, p);
        ODIN_LAUNCH_CHECK();
        const size_t co_smem = (size_t)dk * 32 * sizeof(float) + ((dk & 3) == 0 ? (size_t)CARRY_OUT_TOK * dk * sizeof(float) : 0);
        if (co_smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(recurrence_carry_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)co_smem);
            if (e != cudaSuccess) return (int)e;
        }
        odin_launch(recurrence_carry_out_kernel, dim3(n_items, H, (dv + 31) / 32), dim3(256), co_smem, s, p);
        ODIN_LAUNCH_CHECK();
    }
    return 0;
}

// ------------------------------------------------------------ per-head unit norm, weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[h * w_head_stride + :] * silu(gate[t, h, :])
// One warp per (token, head); the gate and the weight are optional.
template <typename TO>
__global__ void __launch_bounds__(128)
head_unit_scale_kernel(const float* __restrict__ o, const VecRef w, int w_head_stride, const float* __restrict__ gate,
                       long long gate_stride, float eps, TO* __restrict__ out, int T, int H, int dv) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
    ss = warp_sum(ss);
    ss /= (float)dv;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    TO* dst = out + ((size_t)t * H + h) * dv;
    for (int c = lane; c < dv; c += 32) {
        float y = rs * src[c];
        if (w.p != nullptr) y = w.at(h * w_head_stride + c) * y;
        if (gate != nullptr) {
            const float z = gate[(size_t)t * gate_stride + (size_t)h * dv + c];
            y *= z / (1.0f + expf(-z));
        }
        dst[c] = from_f32<TO>(y);
    }
}

extern "C" int odin_head_unit_scale(const float* o, const void* w, int w_dtype, int w_head_stride, const float* gate,
                                    long long gate_stride, float eps, void* out, int out_dtype, int T, int H, int dv,
                                    void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long blocks = ((long long)T * H + 3) / 4;
    if (blocks > 2147483647LL) return ODIN_ERR_UNSUPPORTED;
    VecRef wv{w, w_dtype == ODIN_BF16};
    if (out_dtype == ODIN_BF16)
        odin_launch(head_unit_scale_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, s, o, wv, w_head_stride, gate,
                    gate_stride, eps, (bf16*)out, T, H, dv);
    else if (out_dtype == ODIN_F32)
        odin_launch(head_unit_scale_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, o, wv, w_head_stride, gate,
                    gate_stride, eps, (float*)out, T, H, dv);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}
