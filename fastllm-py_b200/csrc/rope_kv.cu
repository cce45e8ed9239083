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

template <typename T>
__global__ void rope_kv_kernel(T* __restrict__ qkv, long ld, int n_heads, int n_kv_heads,
                               int head_dim, int rot_dim, const float* __restrict__ cos_table,
                               const float* __restrict__ sin_table, const int* __restrict__ positions,
                               const int* __restrict__ slots, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, long page_stride, int page_size,
                               int has_kv) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot_dim >> 1;
    T* row = qkv + (long)t * ld;
    const float* cs = cos_table + (long)pos * half;
    const float* sn = sin_table + (long)pos * half;

    // queries: rotated in place
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, j = idx - h * half;
        T* x = row + (long)h * head_dim;
        const float x1 = to_f32<T>(x[j]), x2 = to_f32<T>(x[j + half]);
        const float c = cs[j], s = sn[j];
        x[j] = from_f32<T>(x1 * c - x2 * s);
        x[j + half] = from_f32<T>(x2 * c + x1 * s);
    }
    if (!has_kv) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const long page = slot / page_size;
    const int off = slot - (int)page * page_size;
    const T* k_in = row + (long)n_heads * head_dim;
    const T* v_in = k_in + (long)n_kv_heads * head_dim;
    T* k_out = k_cache + page * page_stride + (long)off * head_dim;
    T* v_out = v_cache + page * page_stride + (long)off * head_dim;
    const long head_stride = (long)page_size * head_dim;

    // keys: rotated pairs, then the dimensions that are not rotated
    for (int idx = threadIdx.x; idx < n_kv_heads * half; idx += blockDim.x) {
        const int h = idx / half, j = idx - h * half;
        const T* x = k_in + (long)h * head_dim;
        const float x1 = to_f32<T>(x[j]), x2 = to_f32<T>(x[j + half]);
        const float c = cs[j], s = sn[j];
        T* o = k_out + h * head_stride;
        o[j] = from_f32<T>(x1 * c - x2 * s);
        o[j + half] = from_f32<T>(x2 * c + x1 * s);
    }
    const int rest = head_dim - rot_dim;
    for (int idx = threadIdx.x; idx < n_kv_heads * rest; idx += blockDim.x) {
        const int h = idx / rest, j = rot_dim + (idx - h * rest);
        k_out[h * head_stride + j] = k_in[(long)h * head_dim + j];
    }
    // values: copied
    for (int idx = threadIdx.x; idx < n_kv_heads * head_dim; idx += blockDim.x) {
        const int h = idx / head_dim, j = idx - h * head_dim;
        v_out[h * head_stride + j] = v_in[idx];
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
    FL_DISPATCH(dtype, T, (rope_kv_kernel<T><<<n_tokens, 256, 0, stream>>>(
        (T*)qkv, ld, n_heads, n_kv_heads, head_dim, rot_dim, cos_table, sin_table, positions, slots,
        (T*)k_cache, (T*)v_cache, page_stride, page_size, has_kv)));
    return fl_launch_status();
}
