// Paged causal attention on CUDA cores, for any mix of prompt portions and
// single decoded tokens, in bfloat16 or true 32-bit.
//
// One block serves one (token, query head): it walks that token's visible keys
// through the request's block table in tiles of 128 keys, keeps a running
// maximum and sum (softmax in float, exact expf) and accumulates the weighted
// values.  Tiles start at multiples of 128 of the absolute key position, so the
// order of every sum depends only on the token's own position: the result is
// the same bit for bit however the sequence was cut into steps and whatever
// else is in the batch.  This is the reference kernel of the engine: slow,
// simple, and the 32-bit path's attention.
//
// fastllm-py's counterparts: `_sdpa` (fastllm_py/model.py:341-353: scores scaled
// by head_dim^-1/2, keys beyond the query masked, softmax and the weighted sum in
// float) and the decode kernels `attn_decode` (fastllm_py/graph_decode.py:378-420)
// and `battn` (fastllm_py/batched.py:48-92).  Grouped heads are index
// arithmetic, h / (H / KVH), never a materialised repeat (model.py:426-428).
#include "common.cuh"

#define ATT_TILE 128

template <typename T>
__global__ void __launch_bounds__(ATT_TILE) paged_attention_simt_kernel(
    const T* __restrict__ q, long q_ld, T* __restrict__ out, long out_ld,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache, long page_stride, int page_size,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, int n_heads, int n_kv_heads, int head_dim, int window,
    float scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    long* off_s = reinterpret_cast<long*>(smem_raw);                  // [ATT_TILE] element offset of each key row
    float* p_s = reinterpret_cast<float*>(off_s + ATT_TILE);          // [ATT_TILE] softmax numerators of the tile
    float* q_s = p_s + ATT_TILE;                                      // [head_dim]
    __shared__ float scratch[32];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const long head_off = (long)kvh * page_size * head_dim;

    const T* qr = q + (long)t * q_ld + (long)h * head_dim;
    for (int d = tid; d < head_dim; d += ATT_TILE) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    float m = -CUDART_INF_F, l = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
    const int d0 = tid, d1 = tid + ATT_TILE;
    for (int tile = (lo / ATT_TILE) * ATT_TILE; tile <= pos; tile += ATT_TILE) {
        const int j = tile + tid;
        const bool valid = j >= lo && j <= pos;
        float s = -CUDART_INF_F;
        long off = 0;
        if (valid) {
            const long page = bt[j / page_size];
            off = page * page_stride + head_off + (long)(j % page_size) * head_dim;
            const T* kp = k_cache + off;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += q_s[d] * to_f32<T>(kp[d]);
            s = dot * scale;
        }
        off_s[tid] = off;
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = valid ? expf(s - m_new) : 0.0f;
        p_s[tid] = p;
        const float tile_sum = block_sum(p, scratch);     // its barriers also publish p_s / off_s
        const float corr = expf(m - m_new);               // 0 at the first tile (m = -inf)
        l = l * corr + tile_sum;
        const int j_begin = max(0, lo - tile);
        const int j_end = min(ATT_TILE, pos - tile + 1);
        if (d0 < head_dim) {
            float a = acc0 * corr;
            for (int jj = j_begin; jj < j_end; ++jj) a += p_s[jj] * to_f32<T>(v_cache[off_s[jj] + d0]);
            acc0 = a;
        }
        if (d1 < head_dim) {
            float a = acc1 * corr;
            for (int jj = j_begin; jj < j_end; ++jj) a += p_s[jj] * to_f32<T>(v_cache[off_s[jj] + d1]);
            acc1 = a;
        }
        m = m_new;
        __syncthreads();                                  // p_s / off_s are rewritten by the next tile
    }
    T* o = out + (long)t * out_ld + (long)h * head_dim;
    if (d0 < head_dim) o[d0] = from_f32<T>(acc0 / l);
    if (d1 < head_dim) o[d1] = from_f32<T>(acc1 / l);
}

// q: [n_tokens, q_ld] with head h at columns [h*head_dim, (h+1)*head_dim);
// out likewise.  tok_req[t] is the row of `block_table` that token t's request
// uses; positions[t] is the token's absolute position, whose key (already in
// the cache) is the last one it sees.  window <= 0 means all keys.
FL_API int fl_paged_attention_simt(const void* q, int dtype, long q_ld, void* out, long out_ld,
                                   const void* k_cache, const void* v_cache, long page_stride,
                                   int page_size, const int* block_table, int bt_stride,
                                   const int* tok_req, const int* positions, int n_tokens,
                                   int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim < 1 || head_dim > 2 * ATT_TILE || n_heads > 65535 || n_heads % n_kv_heads)
        return (int)cudaErrorInvalidValue;
    const size_t smem = ATT_TILE * (sizeof(long) + sizeof(float)) + (size_t)head_dim * sizeof(float);
    dim3 grid(n_tokens, n_heads);
    FL_DISPATCH(dtype, T, return fl_launch(paged_attention_simt_kernel<T>, grid, dim3(ATT_TILE), smem, stream,
                                           (const T*)q, q_ld, (T*)out, out_ld, (const T*)k_cache,
                                           (const T*)v_cache, page_stride, page_size, block_table, bt_stride,
                                           tok_req, positions, n_heads, n_kv_heads, head_dim, window, scale));
    return 0;
}
