// Sampling on the device: greedy, temperature, top-k, min-p, nucleus (top-p) and
// the three penalties, one block per logits row, so that only token ids go back
// to the host.
//
// fastllm-py samples on the host in float64 (fastllm_py/graph_decode.py:73-133):
// penalties, then softmax(logits / T), then top-k, min-p and top-p, each
// followed by renormalisation, then numpy's Generator.choice, which inverts the
// cumulative distribution with one uniform number.  The same decisions are
// taken here without sorting:
//   * top-k keeps logits >= the k-th largest, found by a radix descent over
//     the logits' bit patterns;
//   * min-p keeps weights >= min_p * (largest weight), and the largest is 1;
//   * top-p keeps a token iff the kept tokens with a larger weight sum to at
//     most top_p of the total (the token that crosses top_p is kept), found by
//     a radix descent over the weights' bit patterns with bin sums;
//   * the draw walks the kept weights in index order until the running sum
//     passes uniform * total.
// Renormalising between the filters changes no decision, so it is done once.
// Bin sums use 2^40 fixed point and integer atomics: their result does not
// depend on the order in which threads arrive, so a row's token depends only on
// its logits, its options and its uniform number.
#include "common.cuh"

#define SAMP_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);      // larger float <=> larger key
}

// (value, index) of the row's maximum, lowest index on ties; every thread gets it.
__device__ void block_argmax(const float* __restrict__ x, int vocab, float* best_val, int* best_idx) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    float v = -CUDART_INF_F;
    int idx = 0x7fffffff;
    // four independent loads per round, so that a row of 100 000 logits does not
    // cost a hundred dependent memory round trips per thread
    int i = threadIdx.x;
    const int stride = blockDim.x;
    for (; i + 3 * stride < vocab; i += 4 * stride) {
        const float a = x[i], b = x[i + stride], c = x[i + 2 * stride], d = x[i + 3 * stride];
        if (a > v || idx == 0x7fffffff) { v = a; idx = i; }
        if (b > v) { v = b; idx = i + stride; }
        if (c > v) { v = c; idx = i + 2 * stride; }
        if (d > v) { v = d; idx = i + 3 * stride; }
    }
    for (; i < vocab; i += stride) {
        const float xi = x[i];
        if (xi > v || idx == 0x7fffffff) { v = xi; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = v; s_idx[warp] = idx; }
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    v = lane < nwarps ? s_val[lane] : -CUDART_INF_F;
    idx = lane < nwarps ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    *best_val = v;
    *best_idx = idx;
}

__device__ __forceinline__ unsigned long long fixed40(float w) {
    return (unsigned long long)((double)w * 1099511627776.0);     // w in [0, 1]
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(
    const float* __restrict__ logits, long ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const double* __restrict__ uniform, int* __restrict__ out) {
    __shared__ unsigned long long hist[256];
    __shared__ unsigned long long s_total;
    __shared__ uint32_t s_prefix;
    __shared__ unsigned long long s_carry;
    __shared__ double s_scan[SAMP_THREADS + 1];
    __shared__ double s_warp[32];

    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (long)row * ld;
    float mx;
    int arg;
    block_argmax(x, vocab, &mx, &arg);
    const float T = temperature ? temperature[row] : 0.0f;
    if (!(T > 0.0f)) {
        if (tid == 0) out[row] = arg;
        return;
    }
    const float inv_t = 1.0f / T;

    // ---- top-k: key of the k-th largest logit
    uint32_t kth_key = 0;
    const int k = top_k ? top_k[row] : 0;
    if (k > 0 && k < vocab) {
        uint32_t prefix = 0, mask = 0;
        unsigned long long remaining = (unsigned long long)k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += SAMP_THREADS) hist[b] = 0;
            __syncthreads();
            for (int i = tid; i < vocab; i += SAMP_THREADS) {
                const uint32_t key = order_key(x[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1ULL);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long rem = remaining;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= rem) break;
                    rem -= hist[b];
                }
                s_prefix = prefix | ((uint32_t)b << shift);
                s_carry = rem;
            }
            __syncthreads();
            prefix = s_prefix;
            remaining = s_carry;
            mask |= 0xffu << shift;
            __syncthreads();
        }
        kth_key = prefix;
    }
    const float mp = min_p ? min_p[row] : 0.0f;
    const float w_floor = mp > 0.0f ? mp : 0.0f;

    // ---- top-p: bit pattern of the smallest kept weight
    uint32_t w_bits_min = 0;
    const float tp = top_p ? top_p[row] : 1.0f;
    if (tp < 1.0f) {
        if (tid == 0) s_total = 0;
        __syncthreads();
        unsigned long long part = 0;
        for (int i = tid; i < vocab; i += SAMP_THREADS) {
            const float xi = x[i];
            const float w = expf((xi - mx) * inv_t);
            if (order_key(xi) >= kth_key && w >= w_floor) part += fixed40(w);
        }
        atomicAdd(&s_total, part);
        __syncthreads();
        const unsigned long long limit = (unsigned long long)((double)tp * (double)s_total);
        uint32_t prefix = 0, mask = 0;
        unsigned long long above = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += SAMP_THREADS) hist[b] = 0;
            __syncthreads();
            for (int i = tid; i < vocab; i += SAMP_THREADS) {
                const float xi = x[i];
                const float w = expf((xi - mx) * inv_t);
                if (order_key(xi) >= kth_key && w >= w_floor) {
                    const uint32_t wb = __float_as_uint(w);
                    if ((wb & mask) == prefix) atomicAdd(&hist[(wb >> shift) & 255u], fixed40(w));
                }
            }
            __syncthreads();
            if (tid == 0) {
                // the lowest bin whose larger-weight mass is still within the limit
                unsigned long long cum = above, chosen_cum = above;
                int chosen = -1;
                for (int b = 255; b >= 0; --b) {
                    if (hist[b] == 0) continue;
                    if (cum <= limit || chosen < 0) { chosen = b; chosen_cum = cum; }
                    else break;
                    cum += hist[b];
                }
                if (chosen < 0) chosen = 0;
                s_prefix = prefix | ((uint32_t)chosen << shift);
                s_carry = chosen_cum;
            }
            __syncthreads();
            prefix = s_prefix;
            above = s_carry;
            mask |= 0xffu << shift;
            __syncthreads();
        }
        w_bits_min = prefix;
    }

    // ---- the draw: first index whose running sum of kept weights passes u * total
    const int chunk = (vocab + SAMP_THREADS - 1) / SAMP_THREADS;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
    double local = 0.0;
    for (int i = begin; i < end; ++i) {
        const float xi = x[i];
        const float w = expf((xi - mx) * inv_t);
        if (order_key(xi) >= kth_key && w >= w_floor && __float_as_uint(w) >= w_bits_min)
            local += (double)w;
    }
    // exclusive scan over the threads' sums
    double incl = local;
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        double v = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double up = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += up;
        }
        s_warp[lane] = v;
    }
    __syncthreads();
    const double warp_base = warp > 0 ? s_warp[warp - 1] : 0.0;
    s_scan[tid + 1] = warp_base + incl;
    if (tid == 0) { s_scan[0] = 0.0; out[row] = arg; }      // the maximum is always kept: a safe default
    __syncthreads();
    const double total = s_scan[SAMP_THREADS];
    const double target = uniform[row] * total;
    const double lo = s_scan[tid], hi = s_scan[tid + 1];
    if (target >= lo && target < hi) {
        double c = lo;
        int pick = -1, last = -1;
        for (int i = begin; i < end; ++i) {
            const float xi = x[i];
            const float w = expf((xi - mx) * inv_t);
            if (order_key(xi) >= kth_key && w >= w_floor && __float_as_uint(w) >= w_bits_min) {
                c += (double)w;
                last = i;
                if (c > target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) out[row] = pick;
    }
}

// logits: [n_rows, ld] float.  Per-row option arrays may be null (no filter;
// a null temperature means greedy for every row).  uniform[row] in [0, 1) is
// used only by rows with temperature > 0.
FL_API int fl_sample(const float* logits, long ld, int n_rows, int vocab, const float* temperature,
                     const int* top_k, const float* top_p, const float* min_p, const double* uniform,
                     int* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    sample_kernel<<<n_rows, SAMP_THREADS, 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p,
                                                      min_p, uniform, out);
    return fl_launch_status();
}

// Penalties over tokens already generated: item i names (row, token, count).
// A positive logit is divided by the row's repetition penalty and a negative one
// multiplied; then frequency * count + presence is subtracted
// (fastllm_py/graph_decode.py:84-92).  Each (row, token) appears at most once.
__global__ void penalties_kernel(float* __restrict__ logits, long ld, const int* __restrict__ rows,
                                 const int* __restrict__ tokens, const int* __restrict__ counts,
                                 int n_items, const float* __restrict__ repetition,
                                 const float* __restrict__ frequency,
                                 const float* __restrict__ presence, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_items) return;
    const int r = rows[i], tok = tokens[i];
    if (tok < 0 || tok >= vocab) return;
    float* p = logits + (long)r * ld + tok;
    float v = *p;
    const float rep = repetition[r];
    if (rep != 1.0f) v = v > 0.0f ? v / rep : v * rep;
    v -= frequency[r] * (float)counts[i] + presence[r];
    *p = v;
}

FL_API int fl_apply_penalties(float* logits, long ld, const int* rows, const int* tokens,
                              const int* counts, int n_items, const float* repetition,
                              const float* frequency, const float* presence, int vocab,
                              cudaStream_t stream) {
    if (n_items <= 0) return 0;
    penalties_kernel<<<(n_items + 255) / 256, 256, 0, stream>>>(logits, ld, rows, tokens, counts,
                                                                n_items, repetition, frequency,
                                                                presence, vocab);
    return fl_launch_status();
}
