// Paged causal attention for prompt portions, bfloat16 on the tensor cores
// (mma.sync m16n8k16), softmax in float.
//
// A CTA of four warps takes 64 consecutive query rows of one request and one
// query head and walks the request's keys in blocks of 64, from the first key
// any of its rows may see to the last, through the block table: keys cached by
// earlier steps and the keys this step wrote are read alike, so a portion of a
// prompt is the same as a whole prompt.  Key blocks start at multiples of 64 of
// the absolute position, so the sequence of partial maxima and sums a row goes
// through depends on the row's position only, not on how the prompt was cut.
// K and V blocks are fetched with cp.async into a two-stage ring while the
// previous block is multiplied.  Scores and the running maximum / sum are
// float; probabilities are rounded to bfloat16 only as the operand of P*V.
//
// fastllm-py's counterpart is `_sdpa` (fastllm_py/model.py:341-353), which
// materialises the (heads, T, S) score tensor with cuBLAS and masks it with
// -1e30; here nothing of size T*S is ever stored.
//
// HEAD_DIM is a compile-time constant (-DHEAD_DIM=...), a multiple of 16 up to 256.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#define ATP_BM 64
#define ATP_BN 64
#define ATP_THREADS 128
#ifndef ATP_STAGES
#define ATP_STAGES 2                      // K/V blocks in shared memory: 2 = fetch the next while multiplying
#endif
#define ATP_DP (HEAD_DIM + 8)              // padded row pitch in shared memory: ldmatrix without bank conflicts
#define ATP_CHUNKS (HEAD_DIM / 8)          // 16-byte chunks per row

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "HEAD_DIM: multiple of 16, at most 256");

__device__ __forceinline__ uint32_t atp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(atp_smem(dst)), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(atp_smem(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(atp_smem(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float atp_weight(float a, float b) {
    return (a == -CUDART_INF_F) ? 0.0f : exp2f(a - b);
}

__global__ void __launch_bounds__(ATP_THREADS) attention_prefill_kernel(
    const bf16* __restrict__ q, long q_ld, bf16* __restrict__ out, long out_ld,
    const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, long page_stride, int page_size,
    int page_shift, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ req_start,
    const int* __restrict__ req_ctx, const int* __restrict__ req_qlen, int n_requests, int include_single,
    int n_heads, int n_kv_heads, int window, float scale_log2e) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char atp_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(atp_raw);                       // [64][DP]
    bf16* Ks = Qs + ATP_BM * ATP_DP;                                   // [stages][64][DP]
    bf16* Vs = Ks + ATP_STAGES * ATP_BN * ATP_DP;                      // [stages][64][DP]

    // which request and which 64-row tile of it this CTA serves (heaviest tiles first)
    int req = -1, tile = 0;
    {
        int acc = 0;
        for (int r = 0; r < n_requests; ++r) {
            const int ql = req_qlen[r];
            const int nt = (ql > 1 || include_single) ? (ql + ATP_BM - 1) / ATP_BM : 0;
            if ((int)blockIdx.x < acc + nt) { req = r; tile = nt - 1 - ((int)blockIdx.x - acc); break; }
            acc += nt;
        }
    }
    if (req < 0) return;
    const int h = blockIdx.y;
    const int kvh = h / (n_heads / n_kv_heads);
    const int q_len = req_qlen[req], ctx = req_ctx[req], row0 = tile * ATP_BM;
    const int tok0 = req_start[req] + row0;
    const int rows_here = min(ATP_BM, q_len - row0);
    const int pos_first = ctx + row0, pos_last = ctx + row0 + rows_here - 1;
    const int lo_tile = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kb_begin = lo_tile / ATP_BN, kb_end = pos_last / ATP_BN + 1;
    const int* bt = block_table + (long)req * bt_stride;
    const long head_off = (long)kvh * page_size * HEAD_DIM;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- loads
    auto load_q = [&]() {
        for (int c = tid; c < ATP_BM * ATP_CHUNKS; c += ATP_THREADS) {
            const int r = c / ATP_CHUNKS, ch = c - r * ATP_CHUNKS;
            const bool real = r < rows_here;
            const bf16* src = q + (long)(tok0 + (real ? r : 0)) * q_ld + (long)h * HEAD_DIM + ch * 8;
            cp_async16(Qs + r * ATP_DP + ch * 8, src, real);
        }
    };
    // Two threads per key row, half of the row's chunks each: one page lookup per thread and block.
    auto load_kv = [&](int kb, int stage) {
        bf16* kd = Ks + stage * ATP_BN * ATP_DP;
        bf16* vd = Vs + stage * ATP_BN * ATP_DP;
        const int r = tid >> 1;
        const int ch0 = (tid & 1) * (ATP_CHUNKS / 2);
        const int j = kb * ATP_BN + r;
        const bool real = j >= lo_tile && j <= pos_last;
        long a = 0;
        if (real) {
            const int pg = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
            const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j - pg * page_size);
            a = (long)bt[pg] * page_stride + head_off + (long)off * HEAD_DIM;
        }
#pragma unroll
        for (int c = 0; c < ATP_CHUNKS / 2; ++c) {
            const int ch = ch0 + c;
            cp_async16(kd + r * ATP_DP + ch * 8, k_cache + a + ch * 8, real);
            cp_async16(vd + r * ATP_DP + ch * 8, v_cache + a + ch * 8, real);
        }
    };

    float o_acc[HEAD_DIM / 8][4];
#pragma unroll
    for (int i = 0; i < HEAD_DIM / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};
    const int g = lane >> 2, tq = lane & 3;
    const int pos_row[2] = {ctx + row0 + warp * 16 + g, ctx + row0 + warp * 16 + g + 8};

    load_q();
    load_kv(kb_begin, 0);
    cp_async_commit();

    for (int kb = kb_begin; kb < kb_end; ++kb) {
#if ATP_STAGES == 2
        const int stage = (kb - kb_begin) & 1;
        if (kb + 1 < kb_end) {
            load_kv(kb + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
#else
        const int stage = 0;
        if (kb > kb_begin) {
            load_kv(kb, 0);
            cp_async_commit();
        }
        cp_async_wait<0>();
#endif
        __syncthreads();
        const bf16* kt = Ks + stage * ATP_BN * ATP_DP;
        const bf16* vt = Vs + stage * ATP_BN * ATP_DP;

        // ---- S = Q K^T for this warp's 16 rows and the block's 64 keys
        float s[ATP_BN / 8][4];
#pragma unroll
        for (int i = 0; i < ATP_BN / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, Qs + (warp * 16 + (lane & 15)) * ATP_DP + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < ATP_BN / 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ATP_DP + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        // ---- scale, mask, running softmax (maxima and sums in units of log2: scores times scale_log2e)
        const int warp_pos_lo = ctx + row0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
        const bool all_seen = (kb * ATP_BN + ATP_BN - 1 <= warp_pos_lo) &&
                              (window <= 0 || kb * ATP_BN > warp_pos_hi - window);
        float corr[2];
        if (all_seen) {
            // every key of the block is visible to every row of this warp: no mask, no special cases
            float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < ATP_BN / 8; ++nt) {
                mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r] * scale_log2e);
                corr[r] = exp2f(m_run[r] - m_new);            // m_new is finite; an empty state gives 0
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nt = 0; nt < ATP_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(fmaf(s[nt][e], scale_log2e, -m_run[e >> 1]));
                    s[nt][e] = p;
                    l_run[e >> 1] += p;
                }
            }
        } else {
            float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < ATP_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = kb * ATP_BN + nt * 8 + 2 * tq + (e & 1);
                    const int pr = pos_row[e >> 1];
                    const bool seen = j <= pr && (window <= 0 || j > pr - window);
                    const float v = seen ? s[nt][e] * scale_log2e : -CUDART_INF_F;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                corr[r] = atp_weight(m_run[r], m_new);
                m_run[r] = m_new;
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int nt = 0; nt < ATP_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = atp_weight(s[nt][e], m_run[e >> 1]);
                    s[nt][e] = p;
                    l_run[e >> 1] += p;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 8; ++i) {
            o_acc[i][0] *= corr[0];
            o_acc[i][1] *= corr[0];
            o_acc[i][2] *= corr[1];
            o_acc[i][3] *= corr[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < ATP_BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HEAD_DIM / 16; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ATP_DP + dp * 16 + (lane >> 4) * 8);
                mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                                    // the stage is refilled two iterations on
    }

    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        if (row >= rows_here) continue;
        const float inv = 1.0f / l_run[r];
        bf16* dst = out + (long)(tok0 + row) * out_ld + (long)h * HEAD_DIM + 2 * tq;
#pragma unroll
        for (int i = 0; i < HEAD_DIM / 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = v;
        }
    }
}

FL_API int fl_attention_prefill_head_dim() { return HEAD_DIM; }

// Every request r of the step with req_qlen[r] > 1 (or >= 1 with include_single)
// gets attention for its rows req_start[r] .. req_start[r] + req_qlen[r] - 1 at
// positions req_ctx[r] + i over its cached keys.  n_tokens bounds the number of
// 64-row tiles.
FL_API int fl_attention_prefill(const void* q, long q_ld, void* out, long out_ld, const void* k_cache,
                                const void* v_cache, long page_stride, int page_size,
                                const int* block_table, int bt_stride, const int* req_start,
                                const int* req_ctx, const int* req_qlen, int n_requests, int n_tokens,
                                int include_single, int n_heads, int n_kv_heads, int window, float scale,
                                cudaStream_t stream) {
    if (n_requests <= 0 || n_tokens <= 0) return 0;
    if (n_heads > 65535 || n_heads % n_kv_heads) return (int)cudaErrorInvalidValue;
    if ((q_ld % 8) || (out_ld % 2) || (page_stride % 8)) return (int)cudaErrorMisalignedAddress;
    const size_t smem = (size_t)(ATP_BM + 2 * ATP_STAGES * ATP_BN) * ATP_DP * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) {
        page_shift = 0;
        while ((1 << page_shift) < page_size) ++page_shift;
    }
    const int max_tiles = n_tokens / ATP_BM + n_requests;   // sum of ceil(q_len / 64) is at most this
    dim3 grid(max_tiles, n_heads);
    return fl_launch(attention_prefill_kernel, grid, dim3(ATP_THREADS), smem, stream, (const bf16*)q, q_ld,
                     (bf16*)out, out_ld, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, page_size,
                     page_shift, block_table, bt_stride, req_start, req_ctx, req_qlen, n_requests,
                     include_single, n_heads, n_kv_heads, window, scale * 1.4426950408889634f);
}
