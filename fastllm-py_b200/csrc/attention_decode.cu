// Split-key paged attention for single decoded tokens, bfloat16, float math.
//
// One query token per request attends to hundreds or thousands of cached keys:
// the work is reading the cache, so the kernel is built to keep many 16-byte
// loads in flight on every SM.  The keys of a token are cut at fixed absolute
// positions (every `split_keys` keys, chosen per launch); one CTA of four warps handles one
// (token, query head, split), each warp a quarter of the split.  Inside a warp a
// key row is spread over HEAD_DIM / 8 lanes (8 bfloat16 = 16 bytes each), so a
// warp covers 32 / lanes-per-key keys per load and eight loads (four keys' worth
// of K and of V per lane group) are issued before any is used.  Scores, the running
// maximum and sum, and the weighted values are float; exp2f on scores pre-scaled
// by log2(e).  Partial (values, maximum, sum) per split go to a float workspace;
// a second kernel merges the splits in ascending order.  Split boundaries and
// the merge order depend on positions only, so a token's result does not depend
// on what else is in the batch.
//
// fastllm-py's counterparts are `attn_decode` (fastllm_py/graph_decode.py:378-420:
// one block per head, all scores in shared memory, hence a context limit) and
// `battn` (fastllm_py/batched.py:48-92: one block per (head, sequence), a block
// reduction per key).  This kernel has no context limit and no per-key barrier.
//
// HEAD_DIM is a compile-time constant (-DHEAD_DIM=...), a multiple of 8 up to 256.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#ifndef ATD_WARPS
#define ATD_WARPS 4
#endif
#ifndef ATD_UNROLL
#define ATD_UNROLL 4
#endif

static_assert(HEAD_DIM % 8 == 0 && HEAD_DIM >= 8 && HEAD_DIM <= 256, "HEAD_DIM: multiple of 8, at most 256");

constexpr int atd_lanes_per_key() {
    int l = 1;
    while (l * 8 < HEAD_DIM) l *= 2;
    return l;
}
constexpr int LPK = atd_lanes_per_key();   // lanes that share one key row (power of two)
constexpr int KPW = 32 / LPK;              // keys a warp reads per load

struct __align__(16) Bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void unpack8(const Bf16x8& p, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// A 16-byte streaming load: the cache is read once per step, so it should not
// displace anything in L1, and neighbouring sectors are worth fetching into L2.
__device__ __forceinline__ Bf16x8 load_stream(const bf16* p) {
    Bf16x8 r;
    uint32_t* w = reinterpret_cast<uint32_t*>(&r);
#ifdef ATD_PLAIN_LOADS
    r = *reinterpret_cast<const Bf16x8*>(p);
#else
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "l"(p));
#endif
    return r;
}

// exp2f(a - b) with the conventions of a running softmax: an empty state (-inf) weighs nothing.
__device__ __forceinline__ float weight_of(float a, float b) {
    return (a == -CUDART_INF_F) ? 0.0f : exp2f(a - b);
}

// workspace rows: [HEAD_DIM values | maximum | sum], one row per (token index, head, split)
#define ATD_ROW (HEAD_DIM + 2)

// out[:] = sum_s values_s * 2^(m_s - M) / sum_s sum_s * 2^(m_s - M) over the splits s_lo..s_hi of one
// (token, head), by one CTA.  Splits are taken ATD_WARPS * 32 at a time with a running maximum, in
// ascending order; the first values of a chunk are requested together with its maxima and sums, so
// that the usual case (a few splits) is one memory round trip.
#define ATD_MERGE_AHEAD 8
#define ATD_MERGE_DPT ((HEAD_DIM + ATD_WARPS * 32 - 1) / (ATD_WARPS * 32))
__device__ __forceinline__ void merge_splits(const float* __restrict__ rows, int s_lo, int s_hi,
                                             bf16* __restrict__ dst) {
    constexpr int NT = ATD_WARPS * 32;
    __shared__ float s_w[NT];
    __shared__ float scratch[32];
    const int tid = threadIdx.x;
    float M = -CUDART_INF_F, L = 0.0f, acc[ATD_MERGE_DPT];
#pragma unroll
    for (int k = 0; k < ATD_MERGE_DPT; ++k) acc[k] = 0.0f;
#pragma unroll 1
    for (int s0 = s_lo; s0 <= s_hi; s0 += NT) {
        const int cnt = min(NT, s_hi - s0 + 1);
        float m_s = -CUDART_INF_F, l_s = 0.0f;
        if (tid < cnt) {
            m_s = __ldcg(rows + (long)(s0 + tid) * ATD_ROW + HEAD_DIM);
            l_s = __ldcg(rows + (long)(s0 + tid) * ATD_ROW + HEAD_DIM + 1);
        }
        float ahead[ATD_MERGE_DPT][ATD_MERGE_AHEAD];
#pragma unroll
        for (int k = 0; k < ATD_MERGE_DPT; ++k) {
            const int d = tid + k * NT;
#pragma unroll
            for (int j = 0; j < ATD_MERGE_AHEAD; ++j)
                ahead[k][j] = (j < cnt && d < HEAD_DIM) ? __ldcg(rows + (long)(s0 + j) * ATD_ROW + d) : 0.0f;
        }
        const float new_m = fmaxf(M, block_max(m_s, scratch));
        s_w[tid] = weight_of(m_s, new_m);
        const float chunk_l = block_sum(l_s * s_w[tid], scratch);           // its barriers publish s_w
        const float corr = weight_of(M, new_m);
        L = L * corr + chunk_l;
#pragma unroll
        for (int k = 0; k < ATD_MERGE_DPT; ++k) {
            const int d = tid + k * NT;
            float a = acc[k] * corr;
#pragma unroll
            for (int j = 0; j < ATD_MERGE_AHEAD; ++j) a += ahead[k][j] * (j < cnt ? s_w[j] : 0.0f);
            if (d < HEAD_DIM)
                for (int j = ATD_MERGE_AHEAD; j < cnt; ++j) a += __ldcg(rows + (long)(s0 + j) * ATD_ROW + d) * s_w[j];
            acc[k] = a;
        }
        M = new_m;
        __syncthreads();                                                    // s_w is rewritten by the next chunk
    }
    const float inv = 1.0f / L;
#pragma unroll
    for (int k = 0; k < ATD_MERGE_DPT; ++k) {
        const int d = tid + k * NT;
        if (d < HEAD_DIM) dst[d] = __float2bfloat16_rn(acc[k] * inv);
    }
}

__global__ void __launch_bounds__(ATD_WARPS * 32) attention_decode_kernel(
    const bf16* __restrict__ q, long q_ld, bf16* __restrict__ out, long out_ld,
    const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, long page_stride, int page_size,
    int page_shift, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, const int* __restrict__ tok_list, int n_heads, int n_kv_heads,
    int window, float scale_log2e, int n_splits, int split_keys, float* __restrict__ partial) {
    pdl_wait();
    pdl_trigger();
    const int li = blockIdx.x;                              // index into the list of decode tokens
    const int t = tok_list ? tok_list[li] : li;
    const int h = blockIdx.y, split = blockIdx.z;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int split_begin = split * split_keys;
    if (split_begin > pos || split_begin + split_keys <= lo) return;       // nothing of this split is visible

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = lane / LPK;                           // which of the warp's KPW keys per load
    const int d0 = (lane % LPK) * 8;                        // this lane's 8 dimensions
    const bool dim_ok = d0 < HEAD_DIM;
    const int kvh = h / (n_heads / n_kv_heads);
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const long head_off = (long)kvh * page_size * HEAD_DIM + d0;

    float qf[8];
    {
        Bf16x8 qv;
        if (dim_ok) qv = *reinterpret_cast<const Bf16x8*>(q + (long)t * q_ld + (long)h * HEAD_DIM + d0);
        else
#pragma unroll
            for (int i = 0; i < 4; ++i) qv.v[i] = __floats2bfloat162_rn(0.0f, 0.0f);
        unpack8(qv, qf);
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[i] *= scale_log2e;
    }

    float m = -CUDART_INF_F, l = 0.0f, o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.0f;

    const int keys_per_warp = split_keys / ATD_WARPS;
    const int warp_begin = split_begin + warp * keys_per_warp;
#pragma unroll 1
    for (int base = warp_begin; base < warp_begin + keys_per_warp; base += KPW * ATD_UNROLL) {
        if (base > pos) break;
        Bf16x8 kv[ATD_UNROLL], vv[ATD_UNROLL];
        bool valid[ATD_UNROLL];
#pragma unroll
        for (int u = 0; u < ATD_UNROLL; ++u) {
            const int j = base + u * KPW + group;
            valid[u] = (j >= lo) && (j <= pos) && (j < warp_begin + keys_per_warp);   // (a round may reach past the warp's keys)
            if (valid[u] && dim_ok) {
                const int pg = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
                const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j - pg * page_size);
                const long a = (long)bt[pg] * page_stride + head_off + (long)off * HEAD_DIM;
                kv[u] = load_stream(k_cache + a);
                vv[u] = load_stream(v_cache + a);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    kv[u].v[i] = __floats2bfloat162_rn(0.0f, 0.0f);
                    vv[u].v[i] = kv[u].v[i];
                }
            }
        }
        float s[ATD_UNROLL];
        float m_new = m;
#pragma unroll
        for (int u = 0; u < ATD_UNROLL; ++u) {
            float kf[8];
            unpack8(kv[u], kf);
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += qf[i] * kf[i];
#pragma unroll
            for (int x = LPK / 2; x > 0; x >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
            s[u] = valid[u] ? dot : -CUDART_INF_F;
            m_new = fmaxf(m_new, s[u]);
        }
        if (m_new != -CUDART_INF_F) {
            const float corr = weight_of(m, m_new);
            l *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] *= corr;
#pragma unroll
            for (int u = 0; u < ATD_UNROLL; ++u) {
                const float p = weight_of(s[u], m_new);
                l += p;
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] += p * vf[i];
            }
            m = m_new;
        }
    }

    // merge the warp's key groups (they saw different keys), in a fixed order
#pragma unroll
    for (int x = LPK; x < 32; x <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, x);
        const float l2 = __shfl_xor_sync(0xffffffffu, l, x);
        const float mm = fmaxf(m, m2);
        const float a1 = weight_of(m, mm), a2 = weight_of(m2, mm);
        l = l * a1 + l2 * a2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float o2 = __shfl_xor_sync(0xffffffffu, o[i], x);
            o[i] = o[i] * a1 + o2 * a2;
        }
        m = mm;
    }
    // merge the four warps through shared memory, warp 0 first
    __shared__ float s_o[ATD_WARPS][LPK * 8];
    __shared__ float s_m[ATD_WARPS], s_l[ATD_WARPS];
    if (lane < LPK) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s_o[warp][lane * 8 + i] = o[i];
        if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
    }
    __syncthreads();
    if (warp == 0 && lane < LPK && dim_ok) {
        float mm = s_m[0];
#pragma unroll
        for (int w = 1; w < ATD_WARPS; ++w) mm = fmaxf(mm, s_m[w]);
        float ll = 0.0f, acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int w = 0; w < ATD_WARPS; ++w) {
            const float a = weight_of(s_m[w], mm);
            ll += s_l[w] * a;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += s_o[w][lane * 8 + i] * a;
        }
        if (n_splits == 1) {
            const float inv = 1.0f / ll;
            bf16* dst = out + (long)t * out_ld + (long)h * HEAD_DIM + d0;
            Bf16x8 r;
#pragma unroll
            for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
            *reinterpret_cast<Bf16x8*>(dst) = r;
        } else {
            float* row = partial + (((long)li * n_heads + h) * n_splits + split) * ATD_ROW;
#pragma unroll
            for (int i = 0; i < 8; ++i) row[d0 + i] = acc[i];
            if (lane == 0) { row[HEAD_DIM] = mm; row[HEAD_DIM + 1] = ll; }
        }
    }
}

// ------------------------------------------------- the tensor-core form
// The same split, but the arithmetic is mma.sync (m16n8k16): the 16 rows of the
// tile are the query heads that share one key/value head (a group of up to 16;
// one real row with plain multi-head attention), so a group's keys and values
// are read once for all its heads, and the dot products, their reductions and
// the weighted sum of the values cost a few dozen warp instructions per 16 keys
// instead of several hundred.  What is left is the stream of the cache: every
// warp owns a quarter of the split's keys, consecutive, and brings them in
// 16 at a time with cp.async through a ring of its own in shared memory (two
// lanes per key row, one page lookup each), so there is no CTA-wide barrier in
// the loop.  Scores, maxima and sums are float; P is rounded to bfloat16 as the
// operand of P V, as in the prompt kernels.  Rows go to the same workspace
// layout as the kernel above writes, and the same merge follows.
#ifndef ATM_CHUNK
#define ATM_CHUNK 16                        // keys per ring stage (a multiple of 16)
#endif
#ifndef ATM_STAGES
#define ATM_STAGES 2
#endif
#define ATM_DP (HEAD_DIM + 8)               // padded row pitch: ldmatrix without bank conflicts
#define ATM_STAGE_ELEMS (ATM_CHUNK * ATM_DP)
#define ATM_WARP_ELEMS (2 * ATM_STAGES * ATM_STAGE_ELEMS)     // K and V stages of one warp
#define ATM_MAX_GROUP 16

__device__ __forceinline__ uint32_t atm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void atm_cp16(void* dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(atm_smem(dst)), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void atm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void atm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void atm_ldmatrix(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(atm_smem(p)));
}
__device__ __forceinline__ void atm_ldmatrix_trans(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(atm_smem(p)));
}
__device__ __forceinline__ void atm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t atm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// grid: (tokens of the list, key/value heads, splits)
__global__ void __launch_bounds__(ATD_WARPS * 32) attention_decode_mma_kernel(
    const bf16* __restrict__ q, long q_ld, bf16* __restrict__ out, long out_ld,
    const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, long page_stride, int page_size,
    int page_shift, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_req,
    const int* __restrict__ positions, const int* __restrict__ tok_list, int n_heads, int n_kv_heads,
    int window, float scale_log2e, int n_splits, int split_keys, float* __restrict__ partial) {
    // What follows up to pdl_wait() reads nothing that the preceding kernels of the step write: the
    // step's tables, and keys and values of EARLIER positions (the kernel before this one writes the
    // cache at the tokens' own positions only).  It runs while that kernel is still at work.
    extern __shared__ __align__(16) unsigned char atm_raw[];
    const int li = blockIdx.x;
    const int t = tok_list ? tok_list[li] : li;
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int group = n_heads / n_kv_heads;                 // query heads per key/value head (<= ATM_MAX_GROUP)
    const int h0 = kvh * group;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int split_begin = split * split_keys;
    if (split_begin > pos || split_begin + split_keys <= lo) return;       // nothing of this split is visible

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;                // fragment coordinates: row (and row + 8), column pair
    const int* bt = block_table + (long)tok_req[t] * bt_stride;
    const long head_off = (long)kvh * page_size * HEAD_DIM;
    bf16* ring = reinterpret_cast<bf16*>(atm_raw) + warp * ATM_WARP_ELEMS;      // [stage][K | V][16][DP]

    // this warp's keys, clipped to what the token sees, in chunks of 16 from the warp's first key
    const int keys_per_warp = split_keys / ATD_WARPS;
    const int warp_begin = split_begin + warp * keys_per_warp;
    const int first = max(warp_begin, lo), last = min(warp_begin + keys_per_warp - 1, pos);
    const int c_begin = first > last ? 0 : (first - warp_begin) / ATM_CHUNK;
    const int c_end = first > last ? 0 : (last - warp_begin) / ATM_CHUNK + 1;

    // Chunk c of this warp into stage (c - c_begin) % ATM_STAGES.  Consecutive lanes take consecutive 16-byte
    // pieces, so one instruction covers whole rows (whole 32-byte sectors); with pages that are a
    // multiple of 16 tokens a chunk lies in one page and is one contiguous piece of K and one of V.
    constexpr int PPR = HEAD_DIM / 8;                       // 16-byte pieces per key row
    const bool chunk_in_page = (page_size % ATM_CHUNK) == 0;
    auto fetch = [&](int c) {
        bf16* kd = ring + ((c - c_begin) % ATM_STAGES) * 2 * ATM_STAGE_ELEMS;
        bf16* vd = kd + ATM_STAGE_ELEMS;
        const int key0 = warp_begin + c * ATM_CHUNK;
        long base = 0;
        if (chunk_in_page) {
            const int pg = page_shift >= 0 ? (key0 >> page_shift) : (key0 / page_size);
            const int off = page_shift >= 0 ? (key0 & (page_size - 1)) : (key0 - pg * page_size);
            base = (long)bt[pg] * page_stride + head_off + (long)off * HEAD_DIM;
        }
#pragma unroll
        for (int x = 0; x < (ATM_CHUNK * PPR + 31) / 32; ++x) {
            const int i = x * 32 + lane;
            const int r = i / PPR, ch = i - r * PPR;
            if ((ATM_CHUNK * PPR) % 32 != 0 && r >= ATM_CHUNK) break;
            const int j = key0 + r;
            const bool real = j >= lo && j <= pos;
            long a = base + (long)r * HEAD_DIM;
            if (!chunk_in_page) {
                a = 0;
                if (real) {
                    const int pg = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
                    const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j - pg * page_size);
                    a = (long)bt[pg] * page_stride + head_off + (long)off * HEAD_DIM;
                }
            }
            atm_cp16(kd + r * ATM_DP + ch * 8, k_cache + a + ch * 8, real);
            atm_cp16(vd + r * ATM_DP + ch * 8, v_cache + a + ch * 8, real);
        }
    };
    // the first chunks: those that end before the token's own position may be asked for at once
    int st = 0;
#pragma unroll
    for (; st < ATM_STAGES; ++st) {
        const int c = c_begin + st;
        if (c >= c_end || warp_begin + c * ATM_CHUNK + ATM_CHUNK - 1 >= pos) break;
        fetch(c);
        atm_commit();
    }
    pdl_wait();
    pdl_trigger();
    for (; st < ATM_STAGES; ++st) {
        if (c_begin + st < c_end) fetch(c_begin + st);
        atm_commit();
    }

    // the queries of the group as the A operand: row = head within the group, zero rows beyond it
    uint32_t qa[HEAD_DIM / 16][4];
    {
        const bf16* q0 = q + (long)t * q_ld + (long)h0 * HEAD_DIM;
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = gq + (e & 1) * 8, col = ks * 16 + 2 * tq + (e >> 1) * 8;
                qa[ks][e] = row < group ? *reinterpret_cast<const uint32_t*>(q0 + (long)row * HEAD_DIM + col) : 0u;
            }
        }
    }

    float o_acc[HEAD_DIM / 8][4];
#pragma unroll
    for (int i = 0; i < HEAD_DIM / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o_acc[i][e] = 0.0f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.0f, 0.0f};

#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
        atm_wait<ATM_STAGES - 1>();                         // chunk c has landed (younger groups may be in flight)
        __syncwarp();
        const bf16* kt = ring + ((c - c_begin) % ATM_STAGES) * 2 * ATM_STAGE_ELEMS;
        const bf16* vt = kt + ATM_STAGE_ELEMS;
        // ---- S = Q K^T: 16 heads x ATM_CHUNK keys
        float sc[ATM_CHUNK / 8][4];
#pragma unroll
        for (int i = 0; i < ATM_CHUNK / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[i][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < ATM_CHUNK / 16; ++np) {
                uint32_t b[4];
                atm_ldmatrix(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ATM_DP + ks * 16 + ((lane >> 3) & 1) * 8);
                atm_mma(sc[2 * np], qa[ks], b[0], b[1]);
                atm_mma(sc[2 * np + 1], qa[ks], b[2], b[3]);
            }
        }
        // ---- running softmax in units of log2 (scores times scale_log2e); keys outside [lo, pos] weigh nothing
        const int key0 = warp_begin + c * ATM_CHUNK;
        const bool all_seen = key0 >= lo && key0 + ATM_CHUNK - 1 <= pos;
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < ATM_CHUNK / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = key0 + nt * 8 + 2 * tq + (e & 1);
                const float v = (all_seen || (j >= lo && j <= pos)) ? sc[nt][e] * scale_log2e : -CUDART_INF_F;
                sc[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = weight_of(m_run[r], m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nt = 0; nt < ATM_CHUNK / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = weight_of(sc[nt][e], m_run[e >> 1]);
                sc[nt][e] = p;
                l_run[e >> 1] += p;
            }
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < HEAD_DIM / 8; ++i) {
                o_acc[i][0] *= corr[0];
                o_acc[i][1] *= corr[0];
                o_acc[i][2] *= corr[1];
                o_acc[i][3] *= corr[1];
            }
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < ATM_CHUNK / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = atm_pack(sc[2 * kk][0], sc[2 * kk][1]);
            pa[1] = atm_pack(sc[2 * kk][2], sc[2 * kk][3]);
            pa[2] = atm_pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
            pa[3] = atm_pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HEAD_DIM / 16; ++dp) {
                uint32_t b[4];
                atm_ldmatrix_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ATM_DP + dp * 16 + (lane >> 4) * 8);
                atm_mma(o_acc[2 * dp], pa, b[0], b[1]);
                atm_mma(o_acc[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();                                       // every lane is done with the stage
        if (c + ATM_STAGES < c_end) fetch(c + ATM_STAGES);
        atm_commit();
    }
    atm_wait<0>();
    // the four lanes of a row hold different keys' sums
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // ---- merge the warps through shared memory (the rings are free now), warp 0 first
    __syncthreads();
    float* s_o = reinterpret_cast<float*>(atm_raw);                     // [warp][head of the group][HEAD_DIM]
    float* s_m = s_o + ATD_WARPS * ATM_MAX_GROUP * HEAD_DIM;            // [warp][head]
    float* s_l = s_m + ATD_WARPS * ATM_MAX_GROUP;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = gq + r * 8;
        if (row < group) {
            float* dst = s_o + ((long)warp * ATM_MAX_GROUP + row) * HEAD_DIM + 2 * tq;
#pragma unroll
            for (int i = 0; i < HEAD_DIM / 8; ++i)
                *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o_acc[i][2 * r], o_acc[i][2 * r + 1]);
            if (tq == 0) {
                s_m[warp * ATM_MAX_GROUP + row] = m_run[r];
                s_l[warp * ATM_MAX_GROUP + row] = l_run[r];
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HEAD_DIM; idx += ATD_WARPS * 32) {
        const int row = idx / HEAD_DIM, d = idx - row * HEAD_DIM;
        float mm = s_m[row];
#pragma unroll
        for (int w = 1; w < ATD_WARPS; ++w) mm = fmaxf(mm, s_m[w * ATM_MAX_GROUP + row]);
        float ll = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < ATD_WARPS; ++w) {
            const float a = weight_of(s_m[w * ATM_MAX_GROUP + row], mm);
            ll += s_l[w * ATM_MAX_GROUP + row] * a;
            acc += s_o[((long)w * ATM_MAX_GROUP + row) * HEAD_DIM + d] * a;
        }
        const int h = h0 + row;
        if (n_splits == 1) {
            out[(long)t * out_ld + (long)h * HEAD_DIM + d] = __float2bfloat16_rn(acc / ll);
        } else {
            float* prow = partial + (((long)li * n_heads + h) * n_splits + split) * ATD_ROW;
            prow[d] = acc;
            if (d == 0) { prow[HEAD_DIM] = mm; prow[HEAD_DIM + 1] = ll; }
        }
    }
}

// The merge kernel: one CTA per (token, head).
__global__ void __launch_bounds__(ATD_WARPS * 32) attention_decode_merge_kernel(
    const float* __restrict__ partial, bf16* __restrict__ out, long out_ld, const int* __restrict__ positions,
    const int* __restrict__ tok_list, int n_heads, int window, int n_splits, int split_keys) {
    const int li = blockIdx.x, h = blockIdx.y;
    const int t = tok_list ? tok_list[li] : li;            // the step's tables: no kernel writes them
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    pdl_wait();
    pdl_trigger();
    merge_splits(partial + ((long)li * n_heads + h) * n_splits * ATD_ROW, lo / split_keys, pos / split_keys,
                 out + (long)t * out_ld + (long)h * HEAD_DIM);
}

FL_API int fl_attention_decode_head_dim() { return HEAD_DIM; }
FL_API int fl_attention_decode_split_unit() { return ATD_WARPS * 16; }    // split sizes are multiples of this
FL_API long fl_attention_decode_workspace_floats(int n_list, int n_heads, int n_splits) {
    return n_splits > 1 ? (long)n_list * n_heads * n_splits * ATD_ROW : 0;
}

// Tokens tok_list[0..n_list) (or 0..n_list when tok_list is null) of q attend to
// their requests' cached keys.  n_splits must cover the longest sequence among
// them: n_splits * split_keys > largest position (split_keys: keys per split, a multiple
// of 64; larger splits stream longer per CTA, smaller ones give more CTAs).  `partial` holds
// fl_attention_decode_workspace_floats(...) floats when n_splits > 1.  `variant`:
// 0 chooses (the tensor-core form when a key/value head serves at most 16 query
// heads), 1 forces the CUDA-core form.
FL_API int fl_attention_decode(const void* q, long q_ld, void* out, long out_ld, const void* k_cache,
                               const void* v_cache, long page_stride, int page_size,
                               const int* block_table, int bt_stride, const int* tok_req,
                               const int* positions, const int* tok_list, int n_list, int n_heads,
                               int n_kv_heads, int window, float scale, int n_splits, int split_keys,
                               float* partial, int variant, cudaStream_t stream) {
    if (n_list <= 0) return 0;
    if (n_heads > 65535 || n_splits < 1 || n_splits > 65535 || n_heads % n_kv_heads) return (int)cudaErrorInvalidValue;
    if (split_keys < ATD_WARPS * 16 || split_keys % (ATD_WARPS * 16)) return (int)cudaErrorInvalidValue;
    if (HEAD_DIM % 16 != 0) variant = 1;
    if ((q_ld % 8) || (out_ld % 8) || (page_stride % 8)) return (int)cudaErrorMisalignedAddress;
    if (n_splits > 1 && partial == nullptr) return (int)cudaErrorInvalidValue;
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) {
        page_shift = 0;
        while ((1 << page_shift) < page_size) ++page_shift;
    }
    int rc;
    if (variant != 1 && n_heads / n_kv_heads <= ATM_MAX_GROUP) {
        // the tensor-core form: one CTA per (token, key/value head, split)
        const size_t ring = (size_t)ATD_WARPS * ATM_WARP_ELEMS * sizeof(bf16);
        const size_t merge = (size_t)ATD_WARPS * ATM_MAX_GROUP * (HEAD_DIM + 2) * sizeof(float);
        const size_t smem = ring > merge ? ring : merge;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        dim3 grid(n_list, n_kv_heads, n_splits);
        rc = fl_launch(attention_decode_mma_kernel, grid, dim3(ATD_WARPS * 32), smem, stream, (const bf16*)q, q_ld,
                       (bf16*)out, out_ld, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, page_size,
                       page_shift, block_table, bt_stride, tok_req, positions, tok_list, n_heads, n_kv_heads,
                       window, scale * 1.4426950408889634f, n_splits, split_keys, partial);
    } else {
        dim3 grid(n_list, n_heads, n_splits);
        rc = fl_launch(attention_decode_kernel, grid, dim3(ATD_WARPS * 32), 0, stream, (const bf16*)q, q_ld,
                       (bf16*)out, out_ld, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, page_size,
                       page_shift, block_table, bt_stride, tok_req, positions, tok_list, n_heads, n_kv_heads,
                       window, scale * 1.4426950408889634f, n_splits, split_keys, partial);
    }
    if (rc || n_splits == 1) return rc;
    dim3 mgrid(n_list, n_heads);
    return fl_launch(attention_decode_merge_kernel, mgrid, dim3(ATD_WARPS * 32), 0, stream, (const float*)partial,
                     (bf16*)out, out_ld, positions, tok_list, n_heads, window, n_splits, split_keys);
}
