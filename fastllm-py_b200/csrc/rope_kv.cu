// Rotary position encoding of queries and keys, fused with the write of the new
// keys and values into the paged cache.
//
// fastllm-py does this in three kernels: `rope` on q, `rope` on k
// (fastllm_py/graph_decode.py:338-357) and `write_kv` / `bwrite_kv`
// (graph_decode.py:432-444, fastllm_py/batched.py:26-40).  Here one kernel reads
// a token's fused q|k|v row once, rotates q in place, and sends the rotated key
// and the value straight to the token's place in its page.
//
// The angles come from a table cos/sin[position, rot_dim/2] that the position
// encoding part builds in float on the host, so the kernel is the same for any
// rotary variant.  Rotate-half pairing: (x[j], x[j + rot_dim/2]); dimensions at
// and beyond rot_dim pass through.
#include "common.cuh"

// One block per (token, head): heads 0 .. n_heads-1 are queries (rotated in
// place), the next n_kv_heads are keys (rotated into the cache), the last
// n_kv_heads are values (copied into the cache).
template <typename T>
__global__ void rope_kv_kernel(T* __restrict__ qkv, long ld, int n_heads, int n_kv_heads,
                               int head_dim, int rot_dim, const float* __restrict__ cos_table,
                               const float* __restrict__ sin_table, const int* __restrict__ positions,
                               const int* __restrict__ slots, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, long page_stride, int page_size) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, head = blockIdx.y;
    const int half = rot_dim >> 1;
    T* x = qkv + (long)t * ld + (long)head * head_dim;
    if (head < n_heads) {
        const long pos = positions[t];
        const float* cs = cos_table + pos * half;
        const float* sn = sin_table + pos * half;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float x1 = to_f32<T>(x[j]), x2 = to_f32<T>(x[j + half]);
            const float c = cs[j], s = sn[j];
            x[j] = from_f32<T>(x1 * c - x2 * s);
            x[j + half] = from_f32<T>(x2 * c + x1 * s);
        }
        return;
    }
    const int slot = slots[t];
    if (slot < 0) return;
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const bool is_key = head < n_heads + n_kv_heads;
    const int kvh = is_key ? head - n_heads : head - n_heads - n_kv_heads;
    T* dst = (is_key ? k_cache : v_cache) + page * page_stride + (long)kvh * page_size * head_dim +
             (long)off * head_dim;
    if (is_key) {
        const long pos = positions[t];
        const float* cs = cos_table + pos * half;
        const float* sn = sin_table + pos * half;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float x1 = to_f32<T>(x[j]), x2 = to_f32<T>(x[j + half]);
            const float c = cs[j], s = sn[j];
            dst[j] = from_f32<T>(x1 * c - x2 * s);
            dst[j + half] = from_f32<T>(x2 * c + x1 * s);
        }
        for (int j = rot_dim + threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = x[j];
    } else {
        for (int j = threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = x[j];
    }
}

// bfloat16, eight elements per thread: a thread takes the pair of 8-element
// vectors (x[j .. j+8), x[j + half .. j + half + 8)) of one head, or one 8-element
// vector of a value head.  Used when head_dim is rotated in full and half is a
// multiple of 8; the form prompt-sized steps use.
__global__ void rope_kv_bf16x8_kernel(bf16* __restrict__ qkv, long ld, int n_heads, int n_kv_heads,
                                      int head_dim, const float* __restrict__ cos_table,
                                      const float* __restrict__ sin_table, const int* __restrict__ positions,
                                      const int* __restrict__ slots, bf16* __restrict__ k_cache,
                                      bf16* __restrict__ v_cache, long page_stride, int page_size,
                                      int has_kv) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int vec_per_head = half >> 3;                         // pairs of vectors per rotated head
    const int rot_heads = n_heads + (has_kv ? n_kv_heads : 0);
    const int rot_items = rot_heads * vec_per_head;
    const int v_items = has_kv ? n_kv_heads * (head_dim >> 3) : 0;
    const int item = blockIdx.y * blockDim.x + threadIdx.x;
    if (item >= rot_items + v_items) return;
    bf16* row = qkv + (long)t * ld;
    long cache_off = 0;
    if (has_kv && item >= n_heads * vec_per_head) {
        const int slot = slots[t];
        if (slot < 0) return;
        const long page = slot / page_size;
        cache_off = page * page_stride + (long)(slot - (int)page * page_size) * head_dim;
    }
    if (item < rot_items) {
        const int head = item / vec_per_head, j = (item - head * vec_per_head) * 8;
        const bf16* x = row + (long)head * head_dim;
        const long pos = positions[t];
        const float* cs = cos_table + pos * half + j;
        const float* sn = sin_table + pos * half + j;
        const uint4 a = *reinterpret_cast<const uint4*>(x + j);
        const uint4 b = *reinterpret_cast<const uint4*>(x + j + half);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        uint4 lo, hi;
        __nv_bfloat162* lp = reinterpret_cast<__nv_bfloat162*>(&lo);
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x1 = __bfloat1622float2(ap[k]), x2 = __bfloat1622float2(bp[k]);
            lp[k] = __floats2bfloat162_rn(x1.x * c[2 * k] - x2.x * sv[2 * k], x1.y * c[2 * k + 1] - x2.y * sv[2 * k + 1]);
            hp[k] = __floats2bfloat162_rn(x2.x * c[2 * k] + x1.x * sv[2 * k], x2.y * c[2 * k + 1] + x1.y * sv[2 * k + 1]);
        }
        bf16* dst = head < n_heads
                        ? row + (long)head * head_dim
                        : k_cache + cache_off + (long)(head - n_heads) * page_size * head_dim;
        *reinterpret_cast<uint4*>(dst + j) = lo;
        *reinterpret_cast<uint4*>(dst + j + half) = hi;
    } else {
        const int vi = item - rot_items;
        const int per = head_dim >> 3;
        const int kvh = vi / per, j = (vi - kvh * per) * 8;
        const bf16* x = row + (long)(n_heads + n_kv_heads + kvh) * head_dim;
        *reinterpret_cast<uint4*>(v_cache + cache_off + (long)kvh * page_size * head_dim + j) =
            *reinterpret_cast<const uint4*>(x + j);
    }
}

// qkv: [n_tokens, ld] rows of q (n_heads*head_dim) | k | v (n_kv_heads*head_dim each);
// when has_kv is 0 the rows hold queries only and nothing is written to a cache.
// k_cache / v_cache point at the key and value halves of a layer's cache
// [page, 2, kv_head, page_size, head_dim]; page_stride counts elements per page.
FL_API int fl_rope_kv_write(void* qkv, int dtype, long ld, int n_tokens, int n_heads,
                            int n_kv_heads, int head_dim, int rot_dim, const float* cos_table,
                            const float* sin_table, const int* positions, const int* slots,
                            void* k_cache, void* v_cache, long page_stride, int page_size,
                            int has_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1)) return (int)cudaErrorInvalidValue;
    const int heads = n_heads + (has_kv ? 2 * n_kv_heads : 0);
    if (heads > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == FL_BF16 && rot_dim == head_dim && head_dim % 16 == 0 && ld % 8 == 0 && page_stride % 8 == 0 &&
        ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 &&
        ((uintptr_t)cos_table % 16) == 0 && ((uintptr_t)sin_table % 16) == 0) {
        const int items = (n_heads + (has_kv ? n_kv_heads : 0)) * (head_dim / 16) +
                          (has_kv ? n_kv_heads * (head_dim / 8) : 0);
        dim3 vgrid(n_tokens, (items + 127) / 128);
        return fl_launch(rope_kv_bf16x8_kernel, vgrid, dim3(128), 0, stream, (bf16*)qkv, ld, n_heads, n_kv_heads,
                         head_dim, cos_table, sin_table, positions, slots, (bf16*)k_cache, (bf16*)v_cache,
                         page_stride, page_size, has_kv);
    }
    dim3 grid(n_tokens, heads);
    const int threads = head_dim >= 128 ? 64 : 32;
    FL_DISPATCH(dtype, T, return fl_launch(rope_kv_kernel<T>, grid, dim3(threads), 0, stream, (T*)qkv, ld,
                                           n_heads, n_kv_heads, head_dim, rot_dim, cos_table, sin_table,
                                           positions, slots, (T*)k_cache, (T*)v_cache, page_stride,
                                           page_size));
    return 0;
}

// The same, reading q|k|v as split-K partial sums (float slabs partial[z][t][col],
// added in the order z = 0, 1, ...) and writing the rotated queries to a buffer
// of the activation type: the product's reduction, the rotation and the cache
// write in one pass.  Each sum is first rounded to the activation type, as the
// separate reduction would have stored it, so both routes give the same bits.
template <typename T>
__global__ void rope_kv_partial_kernel(const float* __restrict__ partial, int splits, long split_stride,
                                       long ld, T* __restrict__ q_out, long q_ld, int n_heads,
                                       int n_kv_heads, int head_dim, int rot_dim,
                                       const float* __restrict__ cos_table,
                                       const float* __restrict__ sin_table,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       T* __restrict__ k_cache, T* __restrict__ v_cache, long page_stride,
                                       int page_size) {
    // Where the token goes and by what angle it turns comes from the step's tables, which no
    // kernel writes: that chain of loads (position -> row of the cos/sin table, slot -> page)
    // runs before the wait for the product, whose partial sums are then all that is left to read.
    const int t = blockIdx.x, head = blockIdx.y;
    const int half = rot_dim >> 1;
    const float* x = partial + (long)t * ld + (long)head * head_dim;
    auto in = [&](int j) {
        float acc = 0.0f;
        for (int z = 0; z < splits; ++z) acc += x[j + (long)z * split_stride];
        return to_f32<T>(from_f32<T>(acc));
    };
    T* dst;
    bool rotate = true;
    if (head < n_heads) {
        dst = q_out + (long)t * q_ld + (long)head * head_dim;
    } else {
        const int slot = slots[t];
        if (slot < 0) return;
        const long page = slot / page_size;
        const int off = slot - (int)page * page_size;
        const bool is_key = head < n_heads + n_kv_heads;
        const int kvh = is_key ? head - n_heads : head - n_heads - n_kv_heads;
        dst = (is_key ? k_cache : v_cache) + page * page_stride + (long)kvh * page_size * head_dim +
              (long)off * head_dim;
        rotate = is_key;
    }
    if (rotate) {
        const long pos = positions[t];
        const float* cs = cos_table + pos * half;
        const float* sn = sin_table + pos * half;
        const int j0 = threadIdx.x;
        float c0 = 1.0f, s0 = 0.0f;                        // this thread's first angle, fetched ahead
        if (j0 < half) { c0 = cs[j0]; s0 = sn[j0]; }
        pdl_wait();
        pdl_trigger();
        for (int j = j0; j < half; j += blockDim.x) {
            const float x1 = in(j), x2 = in(j + half);
            const float c = j == j0 ? c0 : cs[j], s = j == j0 ? s0 : sn[j];
            dst[j] = from_f32<T>(x1 * c - x2 * s);
            dst[j + half] = from_f32<T>(x2 * c + x1 * s);
        }
        for (int j = rot_dim + threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = from_f32<T>(in(j));
    } else {
        pdl_wait();
        pdl_trigger();
        for (int j = threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = from_f32<T>(in(j));
    }
}

FL_API int fl_rope_kv_write_partial(const float* partial, int splits, long split_stride, long ld,
                                    void* q_out, int dtype, long q_ld, int n_tokens, int n_heads,
                                    int n_kv_heads, int head_dim, int rot_dim, const float* cos_table,
                                    const float* sin_table, const int* positions, const int* slots,
                                    void* k_cache, void* v_cache, long page_stride, int page_size,
                                    int has_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1)) return (int)cudaErrorInvalidValue;
    const int heads = n_heads + (has_kv ? 2 * n_kv_heads : 0);
    if (heads > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(n_tokens, heads);
    const int threads = head_dim >= 128 ? 64 : 32;
    FL_DISPATCH(dtype, T, return fl_launch(rope_kv_partial_kernel<T>, grid, dim3(threads), 0, stream, partial,
                                           splits, split_stride, ld, (T*)q_out, q_ld, n_heads, n_kv_heads,
                                           head_dim, rot_dim, cos_table, sin_table, positions, slots,
                                           (T*)k_cache, (T*)v_cache, page_stride, page_size));
    return 0;
}
