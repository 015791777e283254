// Attention through latents: what stands between the down projections and the attention kernels.
//
//   latent_prep    one row of the fused down projection [query latent | key/value latent | rotated key part]:
//                  RMSNorm (with a weight) of the query latent -> its own buffer; RMSNorm of the key/value
//                  latent and the rotation of the key part -> ONE row of the paged cache,
//                  [latent c (kv_rank) | rotated key part (rot)], which serves every head as key AND as value.
//   heads_linear   a product per head: out[t, h, n] = sum_k a[t, h, k] * w[h][k][n].  With w = W_uk of head h it
//                  turns a head's unrotated query into a query over the cached latent (q . (W_uk c) = (W_uk^T q) . c),
//                  with w = W_uv^T of head h the attention's output over the latent into the head's value.
//   rope_heads     rotation of the first `rot` elements of every head by the token's position, pairs (2i, 2i+1) or
//                  (i, i + rot/2), the rest copied; an optional factor on the heads from a given one on.
//
// All arithmetic is 32-bit.  Every output element is one sum in an order that the sizes fix (k ascending in one
// thread; a row's sum of squares by the block's fixed tree), so a token's values do not depend on the batch.
#include "common.cuh"

#define LP_THREADS 128

// cos_t, sin_t: [table_len][rot / 2]; any gain on the rotation is part of the tables.
__device__ __forceinline__ void rotate_pair(float u, float v, float c, float s, float& ru, float& rv) {
    ru = u * c - v * s;
    rv = v * c + u * s;
}

template <typename TI, typename T>
__global__ void __launch_bounds__(LP_THREADS)
latent_prep_kernel(const TI* __restrict__ down, int n_split, size_t split_stride, size_t row_stride, int q_rank,
                   int kv_rank, int rot, int pairs, VecRef qw, VecRef cw, float eps, T* __restrict__ cq,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                   const int* __restrict__ block_table, int bt_stride, T* __restrict__ cache, int page_size,
                   int write_cache) {
    __shared__ float red[32];
    extern __shared__ float rowbuf[];   // q_rank + kv_rank + rot
    pdl_trigger();
    const int t = blockIdx.x;
    const int seq = tok_seq[t];
    const int pos = tok_pos[t];
    int page = -1;
    if (seq >= 0 && write_cache) page = block_table[(size_t)seq * bt_stride + pos / page_size];
    pdl_wait();
    const int n = q_rank + kv_rank + rot;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_split; ++s) v += to_f32(down[(size_t)s * split_stride + (size_t)t * row_stride + j]);
        rowbuf[j] = v;
    }
    __syncthreads();
    if (q_rank > 0) {
        float ss = 0.f;
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x) ss += rowbuf[j] * rowbuf[j];
        ss = block_sum(ss, red);
        ss /= (float)q_rank;
        ss += eps;
        const float rs = 1.0f / sqrtf(ss);
        for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
            cq[(size_t)t * q_rank + j] = from_f32<T>(qw.at(j) * (rs * rowbuf[j]));
    }
    if (page < 0) return;   // padding rows and readers of another entry's line keep nothing
    const float* c = rowbuf + q_rank;
    float ss = 0.f;
    for (int j = threadIdx.x; j < kv_rank; j += blockDim.x) ss += c[j] * c[j];
    ss = block_sum(ss, red);
    ss /= (float)kv_rank;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    T* dst = cache + ((size_t)page * page_size + (pos % page_size)) * (size_t)(kv_rank + rot);
    for (int j = threadIdx.x; j < kv_rank; j += blockDim.x) dst[j] = from_f32<T>(cw.at(j) * (rs * c[j]));
    const float* kr = c + kv_rank;
    const int half = rot / 2;
    const int p = pos < table_len ? pos : table_len - 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int iu = pairs ? 2 * i : i, iv = pairs ? 2 * i + 1 : i + half;
        float ru, rv;
        rotate_pair(kr[iu], kr[iv], cos_t[(size_t)p * half + i], sin_t[(size_t)p * half + i], ru, rv);
        dst[kv_rank + iu] = from_f32<T>(ru);
        dst[kv_rank + iv] = from_f32<T>(rv);
    }
}

extern "C" int odin_latent_prep(const void* down, int in_dtype, int n_split, long long split_stride, long long row_stride,
                                int T, int q_rank, int kv_rank, int rot, int pairs, const void* q_norm, const void* c_norm,
                                int norm_dtype, float eps, void* cq, int out_dtype, const float* cos_t, const float* sin_t,
                                int table_len, const int* tok_pos, const int* tok_seq, const int* block_table,
                                int bt_stride, void* cache, int page_size, int write_cache, void* stream) {
    if (T <= 0) return 0;
    if (q_rank < 0 || kv_rank <= 0 || rot < 0 || (rot & 1) || table_len <= 0) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)(q_rank + kv_rank + rot) * sizeof(float);
    if (smem > 48 * 1024) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef qw{q_norm, norm_dtype == ODIN_BF16}, cw{c_norm, norm_dtype == ODIN_BF16};
#define GO(TI, TT)                                                                                                   \
    odin_launch(latent_prep_kernel<TI, TT>, dim3(T), dim3(LP_THREADS), smem, s, (const TI*)down, n_split,            \
                (size_t)split_stride, (size_t)row_stride, q_rank, kv_rank, rot, pairs, qw, cw, eps, (TT*)cq, cos_t,  \
                sin_t, table_len, tok_pos, tok_seq, block_table, bt_stride, (TT*)cache, page_size, write_cache)
    if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ a product per head
// out[t, h, n] = sum_k a[t, h, k] * w[h][k][n]; a: row stride a_rs, head stride a_hs; out likewise; w: [H][K][N].
// grid (N tiles of HL_THREADS, H, token tiles of HL_TOK); a thread owns one n for HL_TOK tokens and adds over k ascending.
#define HL_THREADS 128
#define HL_TOK 8

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(HL_THREADS)
heads_linear_kernel(const TA* __restrict__ a, size_t a_rs, size_t a_hs, const TW* __restrict__ w, TO* __restrict__ out,
                    size_t o_rs, size_t o_hs, int T, int N, int K) {
    extern __shared__ __align__(16) float as[];   // [K][HL_TOK]
    pdl_trigger();
    const int h = blockIdx.y, t0 = blockIdx.z * HL_TOK;
    const int n = blockIdx.x * HL_THREADS + threadIdx.x;
    pdl_wait();
    for (int e = threadIdx.x; e < K * HL_TOK; e += blockDim.x) {
        const int u = e / K, k = e % K;
        as[k * HL_TOK + u] = (t0 + u < T) ? to_f32(a[(size_t)(t0 + u) * a_rs + (size_t)h * a_hs + k]) : 0.f;
    }
    __syncthreads();
    if (n >= N) return;
    const TW* wh = w + (size_t)h * K * N + n;
    float acc[HL_TOK];
#pragma unroll
    for (int u = 0; u < HL_TOK; ++u) acc[u] = 0.f;
    int k = 0;
    for (; k + 4 <= K; k += 4) {
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = to_f32(wh[(size_t)(k + j) * N]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 a0 = *reinterpret_cast<const float4*>(&as[(k + j) * HL_TOK]);
            const float4 a1 = *reinterpret_cast<const float4*>(&as[(k + j) * HL_TOK + 4]);
            acc[0] = fmaf(wv[j], a0.x, acc[0]); acc[1] = fmaf(wv[j], a0.y, acc[1]);
            acc[2] = fmaf(wv[j], a0.z, acc[2]); acc[3] = fmaf(wv[j], a0.w, acc[3]);
            acc[4] = fmaf(wv[j], a1.x, acc[4]); acc[5] = fmaf(wv[j], a1.y, acc[5]);
            acc[6] = fmaf(wv[j], a1.z, acc[6]); acc[7] = fmaf(wv[j], a1.w, acc[7]);
        }
    }
    for (; k < K; ++k) {
        const float wv = to_f32(wh[(size_t)k * N]);
#pragma unroll
        for (int u = 0; u < HL_TOK; ++u) acc[u] = fmaf(wv, as[k * HL_TOK + u], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < HL_TOK; ++u)
        if (t0 + u < T) out[(size_t)(t0 + u) * o_rs + (size_t)h * o_hs + n] = from_f32<TO>(acc[u]);
}

// Many tokens: a CTA takes 64 tokens by 64 output channels of one head, K in steps of 32 through shared memory, a thread
// four tokens by four channels.  Every output element is the same chain of multiply-adds over k ascending as in the
// kernel above (channels beyond K add exact zeros), so the two give the same bits.
#define HLT_TILE 64
#define HLT_KC 32
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
heads_linear_tiled_kernel(const TA* __restrict__ a, size_t a_rs, size_t a_hs, const TW* __restrict__ w, TO* __restrict__ out,
                          size_t o_rs, size_t o_hs, int T, int N, int K) {
    __shared__ __align__(16) float As[HLT_KC][HLT_TILE + 4];   // [k][token]
    __shared__ __align__(16) float Ws[HLT_KC][HLT_TILE];       // [k][channel]
    pdl_trigger();
    const int h = blockIdx.y, t0 = blockIdx.z * HLT_TILE, n0 = blockIdx.x * HLT_TILE;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const TW* wh = w + (size_t)h * K * N;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    pdl_wait();
    for (int k0 = 0; k0 < K; k0 += HLT_KC) {
        float ra[8], rw[8];
#pragma unroll
        for (int f = 0; f < 8; ++f) {
            const int e = threadIdx.x + f * 256;
            const int u = e / HLT_KC, k = e % HLT_KC;          // a: consecutive threads along k
            ra[f] = (t0 + u < T && k0 + k < K) ? to_f32(a[(size_t)(t0 + u) * a_rs + (size_t)h * a_hs + k0 + k]) : 0.f;
            const int kw = e / HLT_TILE, n = e % HLT_TILE;     // w: consecutive threads along the channels
            rw[f] = (k0 + kw < K && n0 + n < N) ? to_f32(wh[(size_t)(k0 + kw) * N + n0 + n]) : 0.f;
        }
        __syncthreads();   // the step before has been read
#pragma unroll
        for (int f = 0; f < 8; ++f) {
            const int e = threadIdx.x + f * 256;
            As[e % HLT_KC][e / HLT_KC] = ra[f];
            Ws[e / HLT_TILE][e % HLT_TILE] = rw[f];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HLT_KC; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(wv[j], av[i], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) out[(size_t)t * o_rs + (size_t)h * o_hs + n] = from_f32<TO>(acc[i][j]);
        }
    }
}

extern "C" int odin_heads_linear(const void* a, int a_dtype, long long a_rs, long long a_hs, const void* w, int w_dtype,
                                 void* out, int out_dtype, long long o_rs, long long o_hs, int T, int H, int N, int K,
                                 void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 65535 || N <= 0 || K <= 0) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)K * HL_TOK * sizeof(float);
    if (smem > 48 * 1024 || (T + HL_TOK - 1) / HL_TOK > 65535) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)((N + HL_THREADS - 1) / HL_THREADS), (unsigned)H, (unsigned)((T + HL_TOK - 1) / HL_TOK));
    const bool tiled = T >= 32 && (T + HLT_TILE - 1) / HLT_TILE <= 65535;
    const dim3 tgrid((unsigned)((N + HLT_TILE - 1) / HLT_TILE), (unsigned)H, (unsigned)((T + HLT_TILE - 1) / HLT_TILE));
#define GO(TA, TW, TO)                                                                                              \
    do {                                                                                                            \
        if (tiled)                                                                                                  \
            odin_launch(heads_linear_tiled_kernel<TA, TW, TO>, tgrid, dim3(256), 0, s, (const TA*)a, (size_t)a_rs,  \
                        (size_t)a_hs, (const TW*)w, (TO*)out, (size_t)o_rs, (size_t)o_hs, T, N, K);                 \
        else                                                                                                        \
            odin_launch(heads_linear_kernel<TA, TW, TO>, grid, dim3(HL_THREADS), smem, s, (const TA*)a,             \
                        (size_t)a_rs, (size_t)a_hs, (const TW*)w, (TO*)out, (size_t)o_rs, (size_t)o_hs, T, N, K);   \
    } while (0)
    if (a_dtype == ODIN_BF16 && w_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16, bf16);
    else if (a_dtype == ODIN_F32 && w_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float, float);
    else if (a_dtype == ODIN_F32 && w_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(float, bf16, bf16);
    else if (a_dtype == ODIN_BF16 && w_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(bf16, float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ rotation of heads
// For every token t and head h < H: dst[t, h, :width] = rotate(src[t, h, :width]) by tok_pos[t]: the first `rot` elements
// turn (pairs: 2i with 2i+1, else i with i + rot/2), the others are copied; heads h >= scale_from are multiplied by
// `scale` afterwards.  src and dst may be the same memory (every thread reads its elements before it writes them).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rope_heads_kernel(const TI* src, size_t s_rs, size_t s_hs, TO* dst, size_t d_rs, size_t d_hs, int T, int H, int width,
                  int rot, int pairs, float scale, int scale_from, const float* __restrict__ cos_t,
                  const float* __restrict__ sin_t, int table_len, const int* __restrict__ tok_pos) {
    pdl_trigger();
    const int half = rot / 2, per = width - half;   // work items of a head: its pairs, then its other elements
    const long long total = (long long)T * H * per;
    pdl_wait();
    for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(it % per);
        const long long th = it / per;
        const int h = (int)(th % H), t = (int)(th / H);
        const TI* s = src + (size_t)t * s_rs + (size_t)h * s_hs;
        TO* d = dst + (size_t)t * d_rs + (size_t)h * d_hs;
        const float f = h >= scale_from ? scale : 1.0f;
        if (i < half) {
            int p = tok_pos[t];
            p = p < table_len ? (p < 0 ? 0 : p) : table_len - 1;
            const int iu = pairs ? 2 * i : i, iv = pairs ? 2 * i + 1 : i + half;
            float ru, rv;
            rotate_pair(to_f32(s[iu]), to_f32(s[iv]), cos_t[(size_t)p * half + i], sin_t[(size_t)p * half + i], ru, rv);
            d[iu] = from_f32<TO>(ru * f);
            d[iv] = from_f32<TO>(rv * f);
        } else {
            const int e = rot + (i - half);
            d[e] = from_f32<TO>(to_f32(s[e]) * f);
        }
    }
}

extern "C" int odin_rope_heads(const void* src, int s_dtype, long long s_rs, long long s_hs, void* dst, int d_dtype,
                               long long d_rs, long long d_hs, int T, int H, int width, int rot, int pairs, float scale,
                               int scale_from, const float* cos_t, const float* sin_t, int table_len, const int* tok_pos,
                               void* stream) {
    if (T <= 0 || H <= 0 || width <= 0) return 0;
    if (rot < 0 || (rot & 1) || rot > width || (rot > 0 && table_len <= 0)) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)T * H * (width - rot / 2);
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define GO(TI, TO)                                                                                                  \
    odin_launch(rope_heads_kernel<TI, TO>, dim3(blocks), dim3(256), 0, s, (const TI*)src, (size_t)s_rs, (size_t)s_hs, \
                (TO*)dst, (size_t)d_rs, (size_t)d_hs, T, H, width, rot, pairs, scale, scale_from, cos_t, sin_t,       \
                table_len, tok_pos)
    if (s_dtype == ODIN_F32 && d_dtype == ODIN_F32) GO(float, float);
    else if (s_dtype == ODIN_BF16 && d_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (s_dtype == ODIN_F32 && d_dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}
