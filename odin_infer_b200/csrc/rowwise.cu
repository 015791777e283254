// Row kernels of the layers that are not plain RMSNorm + SwiGLU:
//   * the residual update with a norm in groups (the row is cut into equal consecutive parts,
//     each divided by its own root mean square), an optional bias on the update, and the
//     result either normalised (into another buffer or in place) or merely converted;
//   * x += w * (y / rms(y)): an update that is normalised before it is added;
//   * element-wise activations of a product's output (tanh, SiLU, tanh-GELU, xIELU), which add
//     the partial sums of a split product first;
//   * a gate times a row of a per-token table (the product of a gate with a slice of a second
//     embedding).
// All arithmetic is 32-bit; a row's sums run in an order fixed by the block size alone, so a
// row's result does not depend on the other rows of the launch.
#include "common.cuh"

#define ROW_THREADS 256

// ------------------------------------------------------------ residual update + grouped norm
// x_new = x + sum_s delta[s] + bias.  It is written back to x when there is an update and no
// row gather.  mode 0: out = w * (x_new / sqrt(mean_g(x_new^2) + eps)) with the mean over the
// element's own group; out may be x itself (32-bit, in place).  mode 1: out = x_new converted
// (out may be null: the update alone).
// VEC: the row, a group and every distance between rows and parts are multiples of four elements and every
// pointer is 16-byte aligned, so everything moves four elements at a time; the same sums in the same order.
// more: up to two further updates (32-bit, each with parts of its own), added after `delta` in their order.
// scale != 1: the updates and the bias are added up by themselves first, and x_new = x + scale * their sum.
// out2 (mode 0): a second norm of the same x_new with a weight of its own, out2 = w2 * (x_new / rms), the root mean
// square formed once (a block whose two sublayers each read their own norm of one residual stream).
struct MoreDeltas {
    const float* p[2];
    int n_split[2];
    long long stride[2];
    float scale;
    VecRef w2;
    void* out2;
};

template <typename TD, typename TO, bool VEC>
__global__ void __launch_bounds__(ROW_THREADS)
row_update_kernel(float* x, const TD* __restrict__ delta, int n_split, size_t split_stride, VecRef bias, VecRef w,
                  float eps, int groups, int mode, TO* out, const int* __restrict__ rows, int d, MoreDeltas more) {
    __shared__ float red[32];
    extern __shared__ float rowbuf[];  // d floats
    pdl_trigger();
    const int r = blockIdx.x;
    int src = r;
    if (rows != nullptr) src = rows[r];
    pdl_wait();
    TO* o = out == nullptr ? nullptr : out + (size_t)r * d;
    TO* o2 = (mode == 0 && more.out2 != nullptr) ? reinterpret_cast<TO*>(more.out2) + (size_t)r * d : nullptr;
    if (src < 0) {
        if (o != nullptr && (void*)out != (void*)x)
            for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_f32<TO>(0.f);
        if (o2 != nullptr)
            for (int j = threadIdx.x; j < d; j += blockDim.x) o2[j] = from_f32<TO>(0.f);
        return;
    }
    float* xr = x + (size_t)src * d;
    const bool updated = delta != nullptr || bias.p != nullptr || more.p[0] != nullptr || more.p[1] != nullptr;
    const bool write_back = updated && rows == nullptr;
    const bool scaled = more.scale != 1.0f;
    if (VEC) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
            const float4 x0 = ld4(xr + j);
            float4 v = scaled ? make_float4(0.f, 0.f, 0.f, 0.f) : x0;
            if (delta != nullptr)
                for (int s = 0; s < n_split; ++s) {
                    const float4 dv = ld4(delta + (size_t)s * split_stride + (size_t)src * d + j);
                    v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                }
#pragma unroll
            for (int m = 0; m < 2; ++m)
                if (more.p[m] != nullptr)
                    for (int s = 0; s < more.n_split[m]; ++s) {
                        const float4 dv = ld4(more.p[m] + (size_t)s * more.stride[m] + (size_t)src * d + j);
                        v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                    }
            if (bias.p != nullptr) {
                const float4 bv = bias.at4(j);
                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
            }
            if (scaled) v = make_float4(fmaf(more.scale, v.x, x0.x), fmaf(more.scale, v.y, x0.y),
                                        fmaf(more.scale, v.z, x0.z), fmaf(more.scale, v.w, x0.w));
            st4(rowbuf + j, v);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            const float x0 = xr[j];
            float v = scaled ? 0.f : x0;
            if (delta != nullptr)
                for (int s = 0; s < n_split; ++s) v += to_f32(delta[(size_t)s * split_stride + (size_t)src * d + j]);
#pragma unroll
            for (int m = 0; m < 2; ++m)
                if (more.p[m] != nullptr)
                    for (int s = 0; s < more.n_split[m]; ++s) v += more.p[m][(size_t)s * more.stride[m] + (size_t)src * d + j];
            if (bias.p != nullptr) v += bias.at(j);
            if (scaled) v = fmaf(more.scale, v, x0);
            rowbuf[j] = v;
        }
    }
    __syncthreads();
    if (mode == 1) {
        if (VEC) {
            for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
                const float4 v = ld4(rowbuf + j);
                if (write_back) st4(xr + j, v);
                if (o != nullptr) st4(o + j, v);
            }
        } else {
            for (int j = threadIdx.x; j < d; j += blockDim.x) {
                const float v = rowbuf[j];
                if (write_back) xr[j] = v;
                if (o != nullptr) o[j] = from_f32<TO>(v);
            }
        }
        return;
    }
    const int gsz = d / groups;
    const bool keep = write_back && (void*)out != (void*)x;
    for (int g = 0; g < groups; ++g) {
        // a thread adds the squares of its elements in the order of their columns, in both variants
        float ss = 0.f;
        if (VEC) {
            for (int j = threadIdx.x * 4; j < gsz; j += blockDim.x * 4) {
                const float4 v = ld4(rowbuf + g * gsz + j);
                ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
            }
        } else {
            for (int j = threadIdx.x; j < gsz; j += blockDim.x) {
                const float v = rowbuf[g * gsz + j];
                ss += v * v;
            }
        }
        ss = block_sum(ss, red);
        ss /= (float)gsz;
        ss += eps;
        const float rs = 1.0f / sqrtf(ss);
        if (VEC) {
            for (int j = threadIdx.x * 4; j < gsz; j += blockDim.x * 4) {
                const int c = g * gsz + j;
                const float4 v = ld4(rowbuf + c), wv = w.at4(c);
                if (keep) st4(xr + c, v);
                st4(o + c, make_float4(wv.x * (rs * v.x), wv.y * (rs * v.y), wv.z * (rs * v.z), wv.w * (rs * v.w)));
                if (o2 != nullptr) {
                    const float4 w2 = more.w2.at4(c);
                    st4(o2 + c, make_float4(w2.x * (rs * v.x), w2.y * (rs * v.y), w2.z * (rs * v.z), w2.w * (rs * v.w)));
                }
            }
        } else {
            for (int j = threadIdx.x; j < gsz; j += blockDim.x) {
                const int c = g * gsz + j;
                const float v = rowbuf[c];
                if (keep) xr[c] = v;
                o[c] = from_f32<TO>(w.at(c) * (rs * v));
                if (o2 != nullptr) o2[c] = from_f32<TO>(more.w2.at(c) * (rs * v));
            }
        }
    }
}

static int row_update_launch(float* x, const void* delta, int delta_dtype, int n_split, long long split_stride,
                             const void* bias, int bias_dtype, const void* w, int w_dtype, float eps, int groups,
                             int mode, void* out, int out_dtype, const int* rows, int n_rows, int d, MoreDeltas more,
                             void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0 || (mode != 0 && mode != 1)) return ODIN_ERR_BAD_ARG;
    if (mode == 0 && (groups <= 0 || d % groups != 0 || w == nullptr || out == nullptr)) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef wv{w, w_dtype == ODIN_BF16}, bv{bias, bias_dtype == ODIN_BF16};
    const int gsz = mode == 0 ? d / groups : d;
    const bool vec = (d % 4 == 0) && (gsz % 4 == 0) && (split_stride % 4 == 0) && (more.stride[0] % 4 == 0) &&
                     (more.stride[1] % 4 == 0) &&
                     ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)bias) | ((uintptr_t)w) | ((uintptr_t)out) |
                       ((uintptr_t)more.p[0]) | ((uintptr_t)more.p[1]) | ((uintptr_t)more.w2.p) | ((uintptr_t)more.out2)) % 16 == 0);
#define GO(TD, TO)                                                                                               \
    do {                                                                                                         \
        auto kern = vec ? row_update_kernel<TD, TO, true> : row_update_kernel<TD, TO, false>;                    \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != cudaSuccess) return (int)e;                                                                 \
        }                                                                                                        \
        odin_launch(kern, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, (const TD*)delta, n_split,                 \
                    (size_t)split_stride, bv, wv, eps, groups, mode, (TO*)out, rows, d, more);                   \
    } while (0)
    const bool dbf = delta != nullptr && delta_dtype == ODIN_BF16;
    if (out_dtype == ODIN_BF16) { if (dbf) GO(bf16, bf16); else GO(float, bf16); }
    else if (out_dtype == ODIN_F32) { if (dbf) GO(bf16, float); else GO(float, float); }
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

extern "C" int odin_row_update(float* x, const void* delta, int delta_dtype, int n_split, long long split_stride,
                               const void* bias, int bias_dtype, const void* w, int w_dtype, float eps, int groups,
                               int mode, void* out, int out_dtype, const int* rows, int n_rows, int d, void* stream) {
    MoreDeltas more{{nullptr, nullptr}, {0, 0}, {0, 0}, 1.0f, VecRef{nullptr, false}, nullptr};
    return row_update_launch(x, delta, delta_dtype, n_split, split_stride, bias, bias_dtype, w, w_dtype, eps, groups, mode,
                             out, out_dtype, rows, n_rows, d, more, stream);
}

// The same with up to two further 32-bit updates (null: none), each [parts][n, d], added after `delta`, and a factor
// on the sum of all updates (x_new = x + scale * (updates + bias)); and with a second normalised output out2 = w2 * x_new / rms
// (null: none; of out's type, never x itself, with a root mean square over the same groups).
extern "C" int odin_row_update_several(float* x, const void* delta, int delta_dtype, int n_split, long long split_stride,
                                       const float* delta2, int n_split2, long long split_stride2, const float* delta3,
                                       int n_split3, long long split_stride3, const void* bias, int bias_dtype,
                                       const void* w, int w_dtype, float eps, int groups, int mode, void* out,
                                       int out_dtype, const int* rows, int n_rows, int d, float scale, const void* w2,
                                       int w2_dtype, void* out2, void* stream) {
    if (out2 != nullptr && (mode != 0 || w2 == nullptr || out2 == (void*)x || out2 == out)) return ODIN_ERR_BAD_ARG;
    MoreDeltas more{{delta2, delta3}, {n_split2, n_split3}, {split_stride2, split_stride3}, scale,
                    VecRef{w2, w2_dtype == ODIN_BF16}, out2};
    return row_update_launch(x, delta, delta_dtype, n_split, split_stride, bias, bias_dtype, w, w_dtype, eps, groups, mode,
                             out, out_dtype, rows, n_rows, d, more, stream);
}

// ------------------------------------------------------------ x += w * (y / rms(y))
template <typename TY, bool VEC>
__global__ void __launch_bounds__(ROW_THREADS)
normed_add_kernel(float* __restrict__ x, const TY* __restrict__ y, int n_split, size_t split_stride, VecRef w, float eps,
                  const int* __restrict__ tok_seq, int d) {
    __shared__ float red[32];
    extern __shared__ float rowbuf[];
    pdl_trigger();
    const int r = blockIdx.x;
    pdl_wait();
    if (tok_seq != nullptr && tok_seq[r] < 0) return;
    float ss = 0.f;
    if (VEC) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < n_split; ++s) {
                const float4 yv = ld4(y + (size_t)s * split_stride + (size_t)r * d + j);
                v.x += yv.x; v.y += yv.y; v.z += yv.z; v.w += yv.w;
            }
            st4(rowbuf + j, v);
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float v = 0.f;
            for (int s = 0; s < n_split; ++s) v += to_f32(y[(size_t)s * split_stride + (size_t)r * d + j]);
            rowbuf[j] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, red);
    ss /= (float)d;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    float* xr = x + (size_t)r * d;
    if (VEC) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
            const float4 v = ld4(rowbuf + j), wv = w.at4(j);
            float4 xv = ld4(xr + j);
            xv.x += wv.x * (rs * v.x); xv.y += wv.y * (rs * v.y); xv.z += wv.z * (rs * v.z); xv.w += wv.w * (rs * v.w);
            st4(xr + j, xv);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) xr[j] += w.at(j) * (rs * rowbuf[j]);
    }
}

extern "C" int odin_normed_add(float* x, const void* y, int y_dtype, int n_split, long long split_stride, const void* w,
                               int w_dtype, float eps, const int* tok_seq, int n_rows, int d, void* stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    if (d <= 0 || smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef wv{w, w_dtype == ODIN_BF16};
    const bool vec = (d % 4 == 0) && (split_stride % 4 == 0) && ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)w)) % 16 == 0);
#define GO(TY)                                                                                                   \
    do {                                                                                                         \
        auto kern = vec ? normed_add_kernel<TY, true> : normed_add_kernel<TY, false>;                                                                     \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != cudaSuccess) return (int)e;                                                                 \
        }                                                                                                        \
        odin_launch(kern, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, (const TY*)y, n_split, (size_t)split_stride, \
                    wv, eps, tok_seq, d);                                                                        \
    } while (0)
    if (y_dtype == ODIN_BF16) GO(bf16);
    else if (y_dtype == ODIN_F32) GO(float);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ activations
#define ACT_TANH 0
#define ACT_SILU 1
#define ACT_GELU_TANH 2
#define ACT_XIELU 3
#define ACT_RELU2 4

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// xIELU with a_p = softplus(p), a_n = 1/2 + softplus(q):
//   z > 0: a_p z^2 + z/2;   z <= 0: a_n (e^z - 1 - z) + z/2
__device__ __forceinline__ float activate(int act, float z, float c0, float c1) {
    switch (act) {
        case ACT_TANH: return tanhf(z);
        case ACT_SILU: return z / (1.0f + expf(-z));
        case ACT_GELU_TANH: return gelu_tanh_f(z);
        case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
        default: return z > 0.f ? c0 * z * z + 0.5f * z : c1 * (expm1f(z) - z) + 0.5f * z;
    }
}

template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
activation_kernel(const TI* __restrict__ in, int n_split, size_t split_stride, size_t in_stride, int act, VecRef params,
                  TO* __restrict__ out, size_t out_stride, int T, int n, const float* __restrict__ row_scale) {
    pdl_trigger();
    float c0 = 0.f, c1 = 0.f;
    if (act == ACT_XIELU) {
        c0 = softplus_f(params.at(0));
        c1 = 0.5f + softplus_f(params.at(1));
    }
    pdl_wait();
    if (VEC) {  // four elements of a row at a time
        const int n4 = n / 4;
        const long long total4 = (long long)T * n4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
            const int t = (int)(i / n4), c = (int)(i % n4) * 4;
            float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < n_split; ++s) {
                const float4 v = ld4(in + (size_t)s * split_stride + (size_t)t * in_stride + c);
                z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w;
            }
            const float f = row_scale != nullptr ? row_scale[t] : 1.0f;
            st4(out + (size_t)t * out_stride + c, make_float4(activate(act, z.x, c0, c1) * f, activate(act, z.y, c0, c1) * f,
                                                               activate(act, z.z, c0, c1) * f, activate(act, z.w, c0, c1) * f));
        }
        return;
    }
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), c = (int)(i % n);
        float z = 0.f;
        for (int s = 0; s < n_split; ++s) z += to_f32(in[(size_t)s * split_stride + (size_t)t * in_stride + c]);
        out[(size_t)t * out_stride + c] = from_f32<TO>(activate(act, z, c0, c1) * (row_scale != nullptr ? row_scale[t] : 1.0f));
    }
}

extern "C" int odin_activation(const void* in, int in_dtype, int n_split, long long split_stride, long long in_stride,
                               int act, const void* params, int params_dtype, void* out, int out_dtype,
                               long long out_stride, int T, int n, const float* row_scale, void* stream) {
    if (T <= 0 || n <= 0) return 0;
    if (act < 0 || act > ACT_RELU2 || (act == ACT_XIELU && params == nullptr)) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = (n % 4 == 0) && (in_stride % 4 == 0) && (out_stride % 4 == 0) && (split_stride % 4 == 0) &&
                     ((((uintptr_t)in) | ((uintptr_t)out)) % 16 == 0);
    const long long total = (long long)T * n / (vec ? 4 : 1);
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    VecRef pv{params, params_dtype == ODIN_BF16};
#define GO(TI, TO)                                                                                              \
    do {                                                                                                        \
        auto kern = vec ? activation_kernel<TI, TO, true> : activation_kernel<TI, TO, false>;                   \
        odin_launch(kern, dim3(blocks), dim3(256), 0, s, (const TI*)in, n_split,                                \
                    (size_t)split_stride, (size_t)in_stride, act, pv, (TO*)out, (size_t)out_stride, T, n,       \
                    row_scale);                                                                                 \
    } while (0)
    if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_F32) GO(bf16, float);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ gate x row of a per-token table
// out[t, c] = act(sum_s gate[s][t, c]) * table[ids[t], col0 + c]
template <typename TG, typename TT, typename TO>
__global__ void __launch_bounds__(256)
gated_lookup_kernel(const TG* __restrict__ gate, int n_split, size_t split_stride, int act, const TT* __restrict__ table,
                    size_t table_stride, int col0, int V, const int* __restrict__ ids, TO* __restrict__ out, int T, int n) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), c = (int)(i % n);
        const int id = ids[t];
        float z = 0.f;
        for (int s = 0; s < n_split; ++s) z += to_f32(gate[(size_t)s * split_stride + (size_t)t * n + c]);
        const float e = (id >= 0 && id < V) ? to_f32(table[(size_t)id * table_stride + col0 + c]) : 0.f;
        out[(size_t)t * n + c] = from_f32<TO>(activate(act, z, 0.f, 0.f) * e);
    }
}

extern "C" int odin_gated_lookup(const void* gate, int gate_dtype, int n_split, long long split_stride, int act,
                                 const void* table, int table_dtype, long long table_stride, int col0, int V,
                                 const int* ids, void* out, int out_dtype, int T, int n, void* stream) {
    if (T <= 0 || n <= 0) return 0;
    if (act < 0 || act > ACT_GELU_TANH) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)T * n;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define GO(TG, TT, TO)                                                                                          \
    odin_launch(gated_lookup_kernel<TG, TT, TO>, dim3(blocks), dim3(256), 0, s, (const TG*)gate, n_split,       \
                (size_t)split_stride, act, (const TT*)table, (size_t)table_stride, col0, V, ids, (TO*)out, T, n)
    if (gate_dtype == ODIN_F32 && table_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float, float);
    else if (gate_dtype == ODIN_F32 && table_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(float, bf16, bf16);
    else if (gate_dtype == ODIN_BF16 && table_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16, bf16);
    else if (gate_dtype == ODIN_F32 && table_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ gated activation of a gate|up product
// out[t, c] = act(sum_s in[s][t, c]) * (sum_s in[s][t, n + c]) for a product whose row holds the n gate
// columns before the n up columns (SiLU gives SwiGLU, tanh-GELU gives GeGLU); 32-bit arithmetic.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gated_activation_kernel(const TI* __restrict__ in, int n_split, size_t split_stride, size_t in_stride, int act,
                        TO* __restrict__ out, size_t out_stride, int T, int n) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), c = (int)(i % n);
        float g = 0.f, u = 0.f;
        for (int s = 0; s < n_split; ++s) {
            const TI* row = in + (size_t)s * split_stride + (size_t)t * in_stride;
            g += to_f32(row[c]);
            u += to_f32(row[n + c]);
        }
        out[(size_t)t * out_stride + c] = from_f32<TO>(activate(act, g, 0.f, 0.f) * u);
    }
}

extern "C" int odin_gated_activation(const void* in, int in_dtype, int n_split, long long split_stride, long long in_stride,
                                     int act, void* out, int out_dtype, long long out_stride, int T, int n, void* stream) {
    if (T <= 0 || n <= 0) return 0;
    if (act < 0 || act > ACT_GELU_TANH) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)T * n;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define GO(TI, TO)                                                                                                   \
    odin_launch(gated_activation_kernel<TI, TO>, dim3(blocks), dim3(256), 0, s, (const TI*)in, n_split,              \
                (size_t)split_stride, (size_t)in_stride, act, (TO*)out, (size_t)out_stride, T, n)
    if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32) GO(float, float);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16) GO(float, bf16);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16) GO(bf16, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ sigmoid gate on the heads of a mixer's output
// o[t, h * vd + c] *= sigmoid(sum_s gate[s][t, per_head ? h : h * vd + c]): one gate per element, or one per head.
// gate: columns of a (possibly split) product's output, row distance gate_stride; the sigmoid in 32-bit.
template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(TO* __restrict__ o, size_t o_stride, const TG* __restrict__ gate, int n_split, size_t split_stride,
                    size_t gate_stride, int per_head, int T, int H, int vd) {
    pdl_trigger();
    pdl_wait();
    const int n = H * vd;
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n), c = (int)(i % n);
        const int gc = per_head ? c / vd : c;
        float z = 0.f;
        for (int s = 0; s < n_split; ++s) z += to_f32(gate[(size_t)s * split_stride + (size_t)t * gate_stride + gc]);
        TO* p = o + (size_t)t * o_stride + c;
        *p = from_f32<TO>(to_f32(*p) / (1.0f + expf(-z)));
    }
}

// Four elements at a time: vd, every row distance and every pointer are that much aligned.
template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
sigmoid_gate_vec_kernel(TO* __restrict__ o, size_t o_stride, const TG* __restrict__ gate, int n_split, size_t split_stride,
                        size_t gate_stride, int per_head, int T, int H, int vd) {
    pdl_trigger();
    pdl_wait();
    const int n4 = H * vd / 4;
    const long long total = (long long)T * n4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / n4), c = (int)(i % n4) * 4;
        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        if (per_head) {
            float zh = 0.f;
            for (int s = 0; s < n_split; ++s) zh += to_f32(gate[(size_t)s * split_stride + (size_t)t * gate_stride + c / vd]);
            z = make_float4(zh, zh, zh, zh);
        } else {
            for (int s = 0; s < n_split; ++s) {
                const float4 g = ld4(gate + (size_t)s * split_stride + (size_t)t * gate_stride + c);
                z.x += g.x; z.y += g.y; z.z += g.z; z.w += g.w;
            }
        }
        TO* p = o + (size_t)t * o_stride + c;
        const float4 v = ld4(p);
        st4(p, make_float4(v.x / (1.0f + expf(-z.x)), v.y / (1.0f + expf(-z.y)), v.z / (1.0f + expf(-z.z)), v.w / (1.0f + expf(-z.w))));
    }
}

extern "C" int odin_sigmoid_gate(void* o, int o_dtype, long long o_stride, const void* gate, int gate_dtype, int n_split,
                                 long long split_stride, long long gate_stride, int per_head, int T, int H, int vd,
                                 void* stream) {
    if (T <= 0 || H <= 0 || vd <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = (vd % 4 == 0) && (o_stride % 4 == 0) && ((((uintptr_t)o) & 15) == 0) &&
                     (per_head || ((gate_stride % 4 == 0) && (split_stride % 4 == 0) && ((((uintptr_t)gate) & 15) == 0)));
    const long long total = (long long)T * H * vd / (vec ? 4 : 1);
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
#define GO(TG, TO)                                                                                                   \
    do {                                                                                                             \
        auto kern = vec ? sigmoid_gate_vec_kernel<TG, TO> : sigmoid_gate_kernel<TG, TO>;                             \
        odin_launch(kern, dim3(blocks), dim3(256), 0, s, (TO*)o, (size_t)o_stride, (const TG*)gate, n_split,         \
                    (size_t)split_stride, (size_t)gate_stride, per_head, T, H, vd);                                  \
    } while (0)
    if (gate_dtype == ODIN_F32 && o_dtype == ODIN_F32) GO(float, float);
    else if (gate_dtype == ODIN_F32 && o_dtype == ODIN_BF16) GO(float, bf16);
    else if (gate_dtype == ODIN_BF16 && o_dtype == ODIN_BF16) GO(bf16, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ cap and factor on 32-bit values, in place
// z <- scale * cap * tanh(z / cap)   (cap 0: z <- scale * z)
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ z, size_t stride, int rows, int n, float cap,
                                                      float scale) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float* p = z + (size_t)(i / n) * stride + (i % n);
        const float v = cap > 0.f ? cap * tanhf(*p / cap) : *p;
        *p = scale == 1.0f ? v : v * scale;
    }
}

extern "C" int odin_softcap(float* z, long long stride, int rows, int n, float cap, float scale, void* stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (cap < 0.f) return ODIN_ERR_BAD_ARG;
    const long long total = (long long)rows * n;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    odin_launch(softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, z, (size_t)stride, rows, n, cap, scale);
    ODIN_LAUNCH_CHECK();
    return 0;
}


// ------------------------------------------------------------ several terms into one update, normed, added, normed again
// y = sum_i scale_i * rowscale_i[r] * f_i(sum of term i's parts), f_i the identity or w_i * v / rms(v) over the row;
// then x[r] += post_w * y / rms(y) (post_w null: x[r] += y), and out = next_w * x[r] / rms(x[r]) (next_w null: no output).
// Without x the sum itself goes to out as 32-bit values.  rows: gather these rows (x is then left as it is).
// One CTA per row; every sum runs in an order that the width and the block size fix.
#define COMBINE_MAX_TERMS 4
struct CombineTerm {
    const void* p; int is_bf16; int n_split; long long split_stride;
    float scale; const float* row_scale; VecRef norm_w; float norm_eps;
};
struct CombineArgs { CombineTerm t[COMBINE_MAX_TERMS]; int n; };

template <typename TO, bool VEC>
__global__ void __launch_bounds__(ROW_THREADS)
combine_add_kernel(float* __restrict__ x, CombineArgs a, VecRef post_w, float post_eps, VecRef next_w, float next_eps,
                   TO* __restrict__ out, const int* __restrict__ rows, const int* __restrict__ tok_seq, int d) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float cbuf[];
    float* acc = cbuf;        // d
    float* tmp = cbuf + d;    // d
    pdl_trigger();
    const int r = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    pdl_wait();
    if (tok_seq != nullptr && tok_seq[r] < 0) return;
    // VEC: four elements at a time (the width a multiple of four, every row 16-byte aligned); the same sums either way
    constexpr int W = VEC ? 4 : 1;
    const int j0 = threadIdx.x * W, dj = blockDim.x * W;
    auto load = [&](const CombineTerm& tm, size_t at, float* v) {
        if (VEC) {
            const float4 q = tm.is_bf16 ? ld4((const bf16*)tm.p + at) : ld4((const float*)tm.p + at);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
            v[0] = tm.is_bf16 ? __bfloat162float(((const bf16*)tm.p)[at]) : ((const float*)tm.p)[at];
        }
    };
    auto weights = [&](const VecRef& w, int j, float* v) {
        if (VEC) { const float4 q = w.at4(j); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
        else v[0] = w.at(j);
    };
    for (int i = 0; i < a.n; ++i) {
        const CombineTerm& tm = a.t[i];
        float ss = 0.f;
        for (int j = j0; j < d; j += dj) {
            float v[W], u[W];
#pragma unroll
            for (int e = 0; e < W; ++e) v[e] = 0.f;
            for (int sp = 0; sp < tm.n_split; ++sp) {
                load(tm, (size_t)sp * tm.split_stride + (size_t)r * d + j, u);
#pragma unroll
                for (int e = 0; e < W; ++e) v[e] += u[e];
            }
#pragma unroll
            for (int e = 0; e < W; ++e) { tmp[j + e] = v[e]; ss += v[e] * v[e]; }
        }
        float f = tm.scale;
        if (tm.row_scale != nullptr) f *= tm.row_scale[r];
        float rs = 1.0f;
        if (tm.norm_w.p != nullptr) {
            ss = block_sum(ss, red);
            ss /= (float)d;
            ss += tm.norm_eps;
            rs = 1.0f / sqrtf(ss);
        }
        for (int j = j0; j < d; j += dj) {
            float w[W];
            if (tm.norm_w.p != nullptr) weights(tm.norm_w, j, w);
#pragma unroll
            for (int e = 0; e < W; ++e) {
                const float v = tm.norm_w.p != nullptr ? f * (w[e] * (rs * tmp[j + e])) : f * tmp[j + e];
                acc[j + e] = i == 0 ? v : acc[j + e] + v;
            }
        }
    }
    if (x == nullptr) {   // every thread hands on the elements that it summed itself
        for (int j = j0; j < d; j += dj) {
#pragma unroll
            for (int e = 0; e < W; ++e) out[(size_t)blockIdx.x * d + j + e] = from_f32<TO>(acc[j + e]);
        }
        return;
    }
    float rs = 1.0f;
    if (post_w.p != nullptr) {
        float ss = 0.f;
        for (int j = j0; j < d; j += dj) {
#pragma unroll
            for (int e = 0; e < W; ++e) ss += acc[j + e] * acc[j + e];
        }
        ss = block_sum(ss, red);
        ss /= (float)d;
        ss += post_eps;
        rs = 1.0f / sqrtf(ss);
    }
    float* xr = x + (size_t)r * d;
    float s2 = 0.f;
    for (int j = j0; j < d; j += dj) {
        float xv[W], w[W];
        if (VEC) { const float4 q = ld4(xr + j); xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w; }
        else xv[0] = xr[j];
        if (post_w.p != nullptr) weights(post_w, j, w);
#pragma unroll
        for (int e = 0; e < W; ++e) {
            xv[e] += post_w.p != nullptr ? w[e] * (rs * acc[j + e]) : acc[j + e];
            tmp[j + e] = xv[e];
            s2 += xv[e] * xv[e];
        }
        if (rows == nullptr) {
            if (VEC) st4(xr + j, make_float4(xv[0], xv[1], xv[2], xv[3]));
            else xr[j] = xv[0];
        }
    }
    if (next_w.p == nullptr) return;
    s2 = block_sum(s2, red);
    s2 /= (float)d;
    s2 += next_eps;
    const float r2 = 1.0f / sqrtf(s2);
    TO* orow = out + (size_t)blockIdx.x * d;
    for (int j = j0; j < d; j += dj) {
        float w[W];
        weights(next_w, j, w);
        if (VEC) st4(orow + j, make_float4(w[0] * (r2 * tmp[j]), w[1] * (r2 * tmp[j + 1]), w[2] * (r2 * tmp[j + 2]), w[3] * (r2 * tmp[j + 3])));
        else orow[j] = from_f32<TO>(w[0] * (r2 * tmp[j]));
    }
}

extern "C" int odin_combine_add(float* x, int n_terms, const void* const* ptrs, const int* dtypes, const int* n_splits,
                                const long long* split_strides, const float* scales, const float* const* row_scales,
                                const void* const* norm_ws, const int* norm_w_dtypes, const float* norm_eps,
                                const void* post_w, int post_w_dtype, float post_eps, const void* next_w, int next_w_dtype,
                                float next_eps, void* out, int out_dtype, const int* rows, const int* tok_seq, int n_rows,
                                int d, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_terms < 0 || n_terms > COMBINE_MAX_TERMS || d <= 0) return ODIN_ERR_BAD_ARG;
    if (x == nullptr && (out == nullptr || out_dtype != ODIN_F32)) return ODIN_ERR_BAD_ARG;
    if (next_w != nullptr && out == nullptr) return ODIN_ERR_BAD_ARG;
    const size_t smem = (size_t)2 * d * sizeof(float);
    if (smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    CombineArgs a;
    a.n = n_terms;
    uintptr_t all_bits = 0;
    for (int i = 0; i < n_terms; ++i) {
        if (dtypes[i] != ODIN_BF16 && dtypes[i] != ODIN_F32) return ODIN_ERR_UNSUPPORTED;
        a.t[i].p = ptrs[i]; a.t[i].is_bf16 = dtypes[i] == ODIN_BF16; a.t[i].n_split = n_splits[i];
        a.t[i].split_stride = split_strides[i]; a.t[i].scale = scales[i]; a.t[i].row_scale = row_scales[i];
        a.t[i].norm_w = VecRef{norm_ws[i], norm_w_dtypes[i] == ODIN_BF16}; a.t[i].norm_eps = norm_eps[i];
        all_bits |= (uintptr_t)ptrs[i] | (uintptr_t)norm_ws[i] | (uintptr_t)(split_strides[i] * 4);
    }
    all_bits |= (uintptr_t)x | (uintptr_t)out | (uintptr_t)post_w | (uintptr_t)next_w;
    const bool vec = (d % 4 == 0) && (all_bits % 16 == 0);
    cudaStream_t s = (cudaStream_t)stream;
    VecRef pw{post_w, post_w_dtype == ODIN_BF16}, nw{next_w, next_w_dtype == ODIN_BF16};
#define GO(TO)                                                                                                       \
    do {                                                                                                             \
        auto kern = vec ? combine_add_kernel<TO, true> : combine_add_kernel<TO, false>;                              \
        if (smem > 48 * 1024) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
            if (e != cudaSuccess) return (int)e;                                                                     \
        }                                                                                                            \
        odin_launch(kern, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, a, pw, post_eps, nw, next_eps, (TO*)out, rows,   \
                    tok_seq, d);                                                                                     \
    } while (0)
    if (out == nullptr || out_dtype == ODIN_F32) GO(float);
    else if (out_dtype == ODIN_BF16) GO(bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}
