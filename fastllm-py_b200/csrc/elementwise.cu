// Embedding gather, RMSNorm (plain and fused with the residual add) and SwiGLU.
//
// fastllm-py's counterparts: the fancy-index gather `embed[ids]`
// (fastllm_py/model.py:447), `rmsnorm_fused` (fastllm_py/kernels/ops.py:48-68),
// `add_rmsnorm` (fastllm_py/graph_decode.py:300-324) and `swiglu_fused`
// (ops.py:149-153).  As there, all arithmetic is float; sums of squares are
// reduced in an order that depends on the block size only.
#include "common.cuh"

// Four consecutive elements as floats (16-byte loads for float, 8-byte for bfloat16).
__device__ __forceinline__ void load4(const float* p, float4& v) { v = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void load4(const bf16* p, float4& v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v = make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, const float4& v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
// Can rows of `dim` elements of `elem` bytes be read four at a time?
static inline bool vec4_ok(int dim, const void* base, long ld, size_t elem) {
    return base == nullptr || (dim % 4 == 0 && ((uintptr_t)base % (4 * elem)) == 0 && (ld % 4) == 0);
}

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :] as float (the residual stream is float in both
// precisions).  An id outside [0, vocab) writes zeros and records 1 + t in
// *status; it never reads outside the table.  A negative id -1 - r, when `fed`
// is given, stands for fed[r]: a token that an earlier kernel of the stream
// chose (the sampler's output row r) and the host has not read yet.
template <typename TT>
__global__ void embed_kernel(const TT* __restrict__ table, long table_ld, const int* __restrict__ ids,
                             float* __restrict__ out, long out_ld, int hidden, int vocab,
                             int* __restrict__ status, int vec_ok, const int* __restrict__ fed, int n_fed) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && fed != nullptr && -1 - id < n_fed) id = fed[-1 - id];
    float* o = out + (long)t * out_ld;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicCAS(status, 0, t + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const TT* row = table + (long)id * table_ld;
    if (vec_ok) {                                   // hidden % 4 == 0, rows 16-byte aligned
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float4 v;
            load4(row + i, v);
            *reinterpret_cast<float4*>(o + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32<TT>(row[i]);
    }
}

FL_API int fl_embed(const void* table, int table_dtype, long table_ld, const int* ids, float* out,
                    long out_ld, int n_tokens, int hidden, int vocab, int* status, const int* fed, int n_fed,
                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int vec = vec4_ok(hidden, table, table_ld, table_dtype == FL_F32 ? 4 : 2) && vec4_ok(hidden, out, out_ld, 4);
    FL_DISPATCH(table_dtype, TT,
                return fl_launch(embed_kernel<TT>, dim3(n_tokens), dim3(256), 0, stream, (const TT*)table,
                                 table_ld, ids, out, out_ld, hidden, vocab, status, vec, fed, n_fed));
    return 0;
}

// -------------------------------------------------------------------- RMSNorm
// out = x * (mean(x^2) + eps)^-1/2 * w.  With `delta`, first x += delta (x is
// the float residual stream and is written back unless rows are gathered).
// `rows`, when given, selects the input row of each output row.
template <typename TX, typename TD, typename TW, typename TO, bool ADD, bool VEC>
__global__ void rmsnorm_kernel(TX* __restrict__ x, long x_ld, const TD* __restrict__ delta,
                               long delta_ld, const TW* __restrict__ w, TO* __restrict__ out,
                               long out_ld, int dim, float eps, const int* __restrict__ rows,
                               int write_back) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long src = rows ? (long)rows[r] : (long)r;
    TX* xr = x + src * x_ld;
    const TD* dr = ADD ? delta + src * delta_ld : nullptr;
    TO* o = out + (long)r * out_ld;
    constexpr int STEP = VEC ? 4 : 1;
    float ss = 0.0f;
    for (int i = threadIdx.x * STEP; i < dim; i += blockDim.x * STEP) {
        if (VEC) {
            float4 v;
            load4(xr + i, v);
            if (ADD) {
                float4 d;
                load4(dr + i, d);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                if (write_back) store4(xr + i, v);
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        } else {
            float v = to_f32<TX>(xr[i]);
            if (ADD) {
                v += to_f32<TD>(dr[i]);
                if (write_back) xr[i] = from_f32<TX>(v);
            }
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    // Second pass.  With write_back each thread re-reads exactly what it wrote
    // itself; without it the sum is formed again from x and delta.
    const bool readd = ADD && !write_back;
    for (int i = threadIdx.x * STEP; i < dim; i += blockDim.x * STEP) {
        if (VEC) {
            float4 v, g;
            load4(xr + i, v);
            if (readd) {
                float4 d;
                load4(dr + i, d);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            load4(w + i, g);
            store4(o + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        } else {
            float v = to_f32<TX>(xr[i]);
            if (readd) v += to_f32<TD>(dr[i]);
            o[i] = from_f32<TO>(v * inv * to_f32<TW>(w[i]));
        }
    }
}

static inline int norm_threads(int dim, bool vec) {
    int t = vec ? (dim + 3) / 4 : dim;
    t = (t + 31) / 32 * 32;
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

FL_API int fl_rmsnorm(const void* x, int x_dtype, long x_ld, const void* w, int w_dtype, void* out,
                      int out_dtype, long out_ld, int n_rows, int dim, float eps, const int* rows,
                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const bool vec = vec4_ok(dim, x, x_ld, x_dtype == FL_F32 ? 4 : 2) && vec4_ok(dim, w, 4, w_dtype == FL_F32 ? 4 : 2) &&
                     vec4_ok(dim, out, out_ld, out_dtype == FL_F32 ? 4 : 2);
    const int threads = norm_threads(dim, vec);
#define FL_NORM_LAUNCH(VEC)                                                                          \
    FL_DISPATCH(x_dtype, TX, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,                      \
        return fl_launch(rmsnorm_kernel<TX, float, TW, TO, false, VEC>, dim3(n_rows), dim3(threads), 0,  \
                         stream, (TX*)x, x_ld, (const float*)nullptr, 0L, (const TW*)w, (TO*)out,       \
                         out_ld, dim, eps, rows, 0))))
    if (vec) { FL_NORM_LAUNCH(true); } else { FL_NORM_LAUNCH(false); }
#undef FL_NORM_LAUNCH
    return 0;
}

// resid += delta; out = rmsnorm(resid) * w for rows of 4-element chunks, each row by one CTA of 256
// threads that keeps its KEEP chunks per thread in registers across the reduction: every byte is read
// once and written once, all loads of a thread are issued before the first use, and with eight CTAs to
// an SM many rows are in flight.  (The general kernel above reads the row a second time.)
template <typename TD, typename TW, typename TO, int KEEP>
__global__ void __launch_bounds__(256) add_rmsnorm_rows_kernel(float* __restrict__ resid, long resid_ld,
                                                               const TD* __restrict__ delta, long delta_ld,
                                                               const TW* __restrict__ w, TO* __restrict__ out,
                                                               long out_ld, int dim, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* xr = resid + (long)r * resid_ld;
    const TD* dr = delta + (long)r * delta_ld;
    TO* o = out + (long)r * out_ld;
    float4 keep[KEEP], gain[KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < KEEP; ++c) {
        const int i = (threadIdx.x + c * 256) * 4;
        if (i < dim) {
            float4 v = *reinterpret_cast<const float4*>(xr + i), d;
            load4(dr + i, d);
            load4(w + i, gain[c]);
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            *reinterpret_cast<float4*>(xr + i) = v;
            keep[c] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
    for (int c = 0; c < KEEP; ++c) {
        const int i = (threadIdx.x + c * 256) * 4;
        if (i < dim)
            store4(o + i, make_float4(keep[c].x * inv * gain[c].x, keep[c].y * inv * gain[c].y,
                                      keep[c].z * inv * gain[c].z, keep[c].w * inv * gain[c].w));
    }
}

FL_API int fl_add_rmsnorm(float* resid, long resid_ld, const void* delta, int delta_dtype,
                          long delta_ld, const void* w, int w_dtype, void* out, int out_dtype,
                          long out_ld, int n_rows, int dim, float eps, const int* rows,
                          cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int write_back = rows ? 0 : 1;
    if (write_back && dim <= 8 * 1024 && vec4_ok(dim, resid, resid_ld, 4) &&
        vec4_ok(dim, delta, delta_ld, delta_dtype == FL_F32 ? 4 : 2) && vec4_ok(dim, w, 4, w_dtype == FL_F32 ? 4 : 2) &&
        vec4_ok(dim, out, out_ld, out_dtype == FL_F32 ? 4 : 2)) {
        const int chunks = (dim / 4 + 255) / 256;                      // per thread
#define FL_ROWS_LAUNCH(KEEP)                                                                              \
    FL_DISPATCH(delta_dtype, TD, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,                      \
        return fl_launch(add_rmsnorm_rows_kernel<TD, TW, TO, KEEP>, dim3(n_rows), dim3(256), 0, stream,   \
                         resid, resid_ld, (const TD*)delta, delta_ld, (const TW*)w, (TO*)out, out_ld, dim, \
                         eps))))
        if (chunks <= 1) { FL_ROWS_LAUNCH(1); }
        else if (chunks <= 2) { FL_ROWS_LAUNCH(2); }
        else if (chunks <= 4) { FL_ROWS_LAUNCH(4); }
        else { FL_ROWS_LAUNCH(8); }
#undef FL_ROWS_LAUNCH
    }
    const bool vec = vec4_ok(dim, resid, resid_ld, 4) && vec4_ok(dim, delta, delta_ld, delta_dtype == FL_F32 ? 4 : 2) &&
                     vec4_ok(dim, w, 4, w_dtype == FL_F32 ? 4 : 2) && vec4_ok(dim, out, out_ld, out_dtype == FL_F32 ? 4 : 2);
    const int threads = norm_threads(dim, vec);
#define FL_NORM_LAUNCH(VEC)                                                                          \
    FL_DISPATCH(delta_dtype, TD, FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,                  \
        return fl_launch(rmsnorm_kernel<float, TD, TW, TO, true, VEC>, dim3(n_rows), dim3(threads), 0,  \
                         stream, resid, resid_ld, (const TD*)delta, delta_ld, (const TW*)w, (TO*)out,  \
                         out_ld, dim, eps, rows, write_back))))
    if (vec) { FL_NORM_LAUNCH(true); } else { FL_NORM_LAUNCH(false); }
#undef FL_NORM_LAUNCH
    return 0;
}

// resid += delta without a norm (the last pending sum of a stream that ends unnormed).
template <typename TD>
__global__ void add_kernel(float* __restrict__ resid, long resid_ld, const TD* __restrict__ delta,
                           long delta_ld, int dim) {
    pdl_wait();
    pdl_trigger();
    float* xr = resid + (long)blockIdx.x * resid_ld;
    const TD* dr = delta + (long)blockIdx.x * delta_ld;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) xr[i] += to_f32<TD>(dr[i]);
}

FL_API int fl_residual_add(float* resid, long resid_ld, const void* delta, int delta_dtype,
                           long delta_ld, int n_rows, int dim, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    FL_DISPATCH(delta_dtype, TD, return fl_launch(add_kernel<TD>, dim3(n_rows), dim3(256), 0, stream, resid,
                                                  resid_ld, (const TD*)delta, delta_ld, dim));
    return 0;
}

// --------------------------------------------------------------------- SwiGLU
// out[r, i] = silu(gu[r, i]) * gu[r, inter + i]: gate columns first, then up.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, long gu_ld, T* __restrict__ out, long out_ld,
                              int inter) {
    pdl_wait();
    pdl_trigger();
    const T* g = gu + (long)blockIdx.y * gu_ld;
    T* o = out + (long)blockIdx.y * out_ld;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < inter) {
        const float gf = to_f32<T>(g[i]);
        const float uf = to_f32<T>(g[inter + i]);
        o[i] = from_f32<T>(gf / (1.0f + expf(-gf)) * uf);
    }
}

// Eight bfloat16 columns per thread (16-byte loads and stores): the form prompt-sized steps use.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, long gu_ld, bf16* __restrict__ out,
                                     long out_ld, int inter) {
    pdl_wait();
    pdl_trigger();
    const bf16* g = gu + (long)blockIdx.y * gu_ld;
    bf16* o = out + (long)blockIdx.y * out_ld;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= inter) return;
    const uint4 graw = *reinterpret_cast<const uint4*>(g + i);
    const uint4 uraw = *reinterpret_cast<const uint4*>(g + inter + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 res;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
        rp[k] = __floats2bfloat162_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y);
    }
    *reinterpret_cast<uint4*>(o + i) = res;
}

FL_API int fl_swiglu(const void* gu, int dtype, long gu_ld, void* out, long out_ld, int n_rows,
                     int inter, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == FL_BF16 && inter % 8 == 0 && gu_ld % 8 == 0 && out_ld % 8 == 0 &&
        ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        dim3 grid((inter / 8 + 127) / 128, n_rows);
        return fl_launch(swiglu_bf16x8_kernel, grid, dim3(128), 0, stream, (const bf16*)gu, gu_ld, (bf16*)out,
                         out_ld, inter);
    }
    dim3 grid((inter + 255) / 256, n_rows);
    FL_DISPATCH(dtype, T, return fl_launch(swiglu_kernel<T>, grid, dim3(256), 0, stream, (const T*)gu, gu_ld,
                                           (T*)out, out_ld, inter));
    return 0;
}

// ------------------------------------------- consumers of split-K partial sums
// A product whose K was split over CTAs leaves `splits` float slabs
// partial[z][row][col] (slab stride `split_stride`, row pitch `ld`).  Instead of
// a kernel that only adds the slabs, the kernel that consumes the product adds
// them as it reads: in the order z = 0, 1, ..., so the sum is the same as the
// separate reduction's.

__device__ __forceinline__ float sum_splits(const float* __restrict__ p, long idx, int splits,
                                            long split_stride) {
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) acc += p[idx + (long)z * split_stride];
    return acc;
}

// resid[r] += sum_z partial[z][r]; out[r] = rmsnorm(resid[r]) * w
template <typename TW, typename TO>
__global__ void add_rmsnorm_partial_kernel(float* __restrict__ resid, long resid_ld,
                                           const float* __restrict__ partial, int splits,
                                           long split_stride, long ld, const TW* __restrict__ w,
                                           TO* __restrict__ out, long out_ld, int dim, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* xr = resid + (long)r * resid_ld;
    const float* pr = partial + (long)r * ld;
    TO* o = out + (long)r * out_ld;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        // the sum is rounded to the activation type first, as the separate reduction stores it
        const float v = xr[i] + to_f32<TO>(from_f32<TO>(sum_splits(pr, i, splits, split_stride)));
        xr[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        o[i] = from_f32<TO>(xr[i] * inv * to_f32<TW>(w[i]));
}

// The same for rows made of 4-element chunks (dim and every pitch a multiple of
// 4, 16-byte aligned bases) of at most ARP_KEEP chunks per thread.  A decode
// step has a handful of rows, so this kernel is one CTA per row and its time is
// the length of its chain of dependent memory round trips: every load (all slabs,
// the residual, the norm weight) is issued before the first use, the row stays
// in registers across the reduction, and nothing is read a second time.
#define ARP_KEEP 2
template <typename TW, typename TO>
__global__ void __launch_bounds__(1024) add_rmsnorm_partial_vec_kernel(
    float* __restrict__ resid, long resid_ld, const float* __restrict__ partial, int splits, long split_stride,
    long ld, const TW* __restrict__ w, TO* __restrict__ out, long out_ld, int dim, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* xr = resid + (long)r * resid_ld;
    const float* pr = partial + (long)r * ld;
    TO* o = out + (long)r * out_ld;
    float4 keep[ARP_KEEP], gain[ARP_KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < ARP_KEEP; ++c) {
        const int i = (threadIdx.x + c * blockDim.x) * 4;
        if (i < dim) {
            float4 v = *reinterpret_cast<const float4*>(xr + i);
            load4(w + i, gain[c]);
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
            for (int z = 0; z < splits; ++z) {
                const float4 p = *reinterpret_cast<const float4*>(pr + i + (long)z * split_stride);
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            // the sum is rounded to the activation type first, as the separate reduction stores it
            v.x += to_f32<TO>(from_f32<TO>(acc.x));
            v.y += to_f32<TO>(from_f32<TO>(acc.y));
            v.z += to_f32<TO>(from_f32<TO>(acc.z));
            v.w += to_f32<TO>(from_f32<TO>(acc.w));
            *reinterpret_cast<float4*>(xr + i) = v;
            keep[c] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
    for (int c = 0; c < ARP_KEEP; ++c) {
        const int i = (threadIdx.x + c * blockDim.x) * 4;
        if (i < dim)
            store4(o + i, make_float4(keep[c].x * inv * gain[c].x, keep[c].y * inv * gain[c].y,
                                      keep[c].z * inv * gain[c].z, keep[c].w * inv * gain[c].w));
    }
}

FL_API int fl_add_rmsnorm_partial(float* resid, long resid_ld, const float* partial, int splits,
                                  long split_stride, long ld, const void* w, int w_dtype, void* out,
                                  int out_dtype, long out_ld, int n_rows, int dim, float eps,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const bool vec = vec4_ok(dim, resid, resid_ld, 4) && vec4_ok(dim, partial, ld, 4) && split_stride % 4 == 0 &&
                     vec4_ok(dim, w, 4, w_dtype == FL_F32 ? 4 : 2) &&
                     vec4_ok(dim, out, out_ld, out_dtype == FL_F32 ? 4 : 2) && dim <= ARP_KEEP * 4 * 1024;
    if (vec) {
        const int vthreads = dim / 4 <= 1024 ? (dim / 4 + 31) / 32 * 32 : 1024;  // one chunk per thread when that fits
        FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,
            return fl_launch(add_rmsnorm_partial_vec_kernel<TW, TO>, dim3(n_rows), dim3(vthreads), 0, stream,
                             resid, resid_ld, partial, splits, split_stride, ld, (const TW*)w, (TO*)out, out_ld,
                             dim, eps)));
    }
    const int threads = norm_threads(dim, false);
    FL_DISPATCH(w_dtype, TW, FL_DISPATCH(out_dtype, TO,
        return fl_launch(add_rmsnorm_partial_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, resid,
                         resid_ld, partial, splits, split_stride, ld, (const TW*)w, (TO*)out, out_ld, dim,
                         eps)));
    return 0;
}

// out[r, i] = silu(sum_z partial[z][r][i]) * sum_z partial[z][r][inter + i]
template <typename TO>
__global__ void swiglu_partial_kernel(const float* __restrict__ partial, int splits, long split_stride,
                                      long ld, TO* __restrict__ out, long out_ld, int inter) {
    pdl_wait();
    pdl_trigger();
    const float* g = partial + (long)blockIdx.y * ld;
    TO* o = out + (long)blockIdx.y * out_ld;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < inter) {
        // what the separate reduction would have stored, so that both routes agree
        const float gf = to_f32<TO>(from_f32<TO>(sum_splits(g, i, splits, split_stride)));
        const float uf = to_f32<TO>(from_f32<TO>(sum_splits(g, inter + i, splits, split_stride)));
        o[i] = from_f32<TO>(gf / (1.0f + expf(-gf)) * uf);
    }
}

FL_API int fl_swiglu_partial(const float* partial, int splits, long split_stride, long ld, void* out,
                             int out_dtype, long out_ld, int n_rows, int inter, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    dim3 grid((inter + 255) / 256, n_rows);
    FL_DISPATCH(out_dtype, TO, return fl_launch(swiglu_partial_kernel<TO>, grid, dim3(256), 0, stream, partial,
                                                splits, split_stride, ld, (TO*)out, out_ld, inter));
    return 0;
}
