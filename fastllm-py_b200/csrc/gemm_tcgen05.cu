// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 with float accumulation on the
// Blackwell tensor cores: TMA loads into 128-byte-swizzled shared memory,
// tcgen05.mma issued by one thread, the accumulator in tensor memory, read back
// with tcgen05.ld.
//
// fastllm-py leaves this product to cuBLAS (`x @ w.T`, fastllm_py/model.py:63)
// and, for INT4, to Marlin; its own note on decoding is that M = 1 wants a
// GEMV-shaped kernel and not a GEMM tile (fastllm_py/graph_decode.py:541-543).
// This kernel covers both ends with one shape: the WEIGHTS are the 128-row
// operand of the MMA and the TOKENS are its N dimension (16 to 256 wide), so a
// decode step of a few tokens wastes no tensor-core rows and streams each weight
// once, and a prompt portion uses 128 x 256 tiles.  When there are too few tiles
// to keep every SM pulling bytes, K is split over CTAs; partial sums go to a
// float workspace and a second kernel adds them in a fixed order.
//
// The weights come in one of two layouts.  Row-major [N, K] (what a checkpoint has): a stage's weight tile is
// 128 rows x 128 bytes taken from rows a whole K apart, so DRAM serves it 128 bytes at a time from 128 pages.
// Packed by k-block, [ceil(K / 64)][N][64] (`fl_pack_weight` makes it, once, at load): the same tile is 16 KB in
// one piece.  The kernels are the same; only the tile's coordinates differ (`wp`: the rows of a k-block, 0 for
// row-major).  Streaming products run 4 to 7 % faster from the packed layout (6.0 against 5.75 TB/s for the
// q|k|v product of a batch-8 decode step, 7.0 against 6.65 for the vocabulary product).
//
// Roles in a CTA of 192 threads: warp 0 (one lane) issues the TMA loads, warp 1
// owns the tensor memory and (one lane) issues the MMAs, warps 2-5 move the
// accumulator from tensor memory to global memory.  Every wait on an mbarrier is
// bounded: when a wait runs out the CTA records an error code in *status, all
// roles leave their loops, the tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128            // weight rows (output features) per CTA tile
#define TC_BK 64             // K elements per stage: 128 bytes of bfloat16, one swizzle row
#define TC_THREADS 192
#define TC_WAIT_LIMIT_NS 2000000000ull

enum { TC_ERR_FULL_WAIT = 101, TC_ERR_EMPTY_WAIT = 102, TC_ERR_ACC_WAIT = 103 };

// ------------------------------------------------------------------ PTX wraps
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the barrier's phase `parity` to complete.  Gives up (returns false)
// when another role has already given up or after TC_WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > TC_WAIT_LIMIT_NS) return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// silu(g) * u with the fast exponential and division: the epilogue has a fixed budget per tile (the
// next tile's MMAs), and the exact forms cost five times the instructions for digits that a
// bfloat16 result cannot hold (relative error about 1e-6 against bfloat16's 4e-3).
__device__ __forceinline__ float gated_act(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// A barrier among the four epilogue warps only (hardware barrier 1; barrier 0 is __syncthreads).
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 bfloat16) in the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                     // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                     // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: float accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// Rows of 128 (or fewer) values from the epilogue's staging area to global memory, 16 bytes per
// thread where the destination allows it: `e` is the thread's index among the 128 epilogue threads,
// `cols` how many of the 128 columns exist.  Written this way a warp stores whole rows of 256 or 512
// bytes; one value per lane and row (what the accumulator's layout gives) took 40 ns per token.
template <typename T, int WIDTH, int ROWS = 32>
__device__ __forceinline__ void tc_copy_rows(T* __restrict__ dst, long ld, const T* __restrict__ src, int rows,
                                             int cols, int e, bool vec_ok) {
    constexpr int V = 16 / (int)sizeof(T);                  // values per 16 bytes
    constexpr int TPR = WIDTH / V;                          // threads per row
    constexpr int RPP = 128 / TPR;                          // rows per pass
    const int rr = e / TPR, cc = (e % TPR) * V;
#pragma unroll
    for (int p = 0; p < (ROWS + RPP - 1) / RPP; ++p) {
        const int row = p * RPP + rr;
        if (row >= rows || cc >= cols) continue;
        T* d = dst + (long)row * ld + cc;
        const T* s_ = src + row * WIDTH + cc;
        if (vec_ok && cc + V <= cols) {
            *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s_);
        } else {
            for (int v = 0; v < V && cc + v < cols; ++v) d[v] = s_[v];
        }
    }
}
#define TC2_PEER_MASK 0xFEFFFFFFu                          // clears the CTA-rank bit of a shared::cluster address

template <int BN, int STAGES>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * TC_BK * 2;
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int MAX_STAGES = 12;                         // (the gated form makes its stages at run time)
    static constexpr int BAR_BYTES = (2 * MAX_STAGES + 1) * 8 + 16;
    static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;   // slack to align the tiles to 1024
};

// grid: (ceil(N / 128), ceil(M / BN), splits).  OutT: the type of C when
// splits == 1; with splits > 1 float partial sums go to `partial[z][M][ld_partial]`.
//
// GATED (the SwiGLU feed-forward's first product, no K split): W holds the gate rows and, `gate_rows`
// further down, the up rows; a CTA serves `feat` features (a multiple of 8 up to 64): its weight tile
// is `feat` gate rows and below them the `feat` up rows of the same features (two TMA boxes of `feat`
// rows: map_w has such boxes then), N counts features, and the epilogue writes silu(gate) * up: the
// product's 2 x N columns never go to memory.  The MMA still reads 128 rows: those past 2 x feat are
// whatever lies behind the tile in shared memory and end in accumulator rows that nobody reads.  The
// launcher picks `feat` so that all CTAs fit the SMs at once (two per SM); a stage is then smaller and
// the ring has more of them, which is what keeps enough loads in flight: 172 CTAs of 64 features
// streamed DeepSeek-7B's gate|up weights at 5.3 TB/s inside a decode step.
template <int BN, int STAGES, typename OutT, bool GATED>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
    OutT* __restrict__ C, long ldc, float* __restrict__ partial, long ld_partial, int M, int N, int K,
    int kb_per_split, int* __restrict__ status, int gate_rows, int feat, int wp) {
    using L = TcSmem<BN, STAGES>;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + L::TILE_BYTES);
    uint64_t* empty_bar = full_bar + L::MAX_STAGES;
    uint64_t* acc_bar = empty_bar + L::MAX_STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // a stage: the weight rows, then the token rows.  GATED: 2 x feat weight rows, and as many stages as
    // leave the last one 128 rows of room for the MMA to read
    const int w_bytes = GATED ? feat * 2 * TC_BK * 2 : L::A_BYTES;
    const int stage_bytes = w_bytes + L::B_BYTES;
    const int n_stages = GATED ? min(L::MAX_STAGES, (L::TILE_BYTES - L::A_BYTES - L::B_BYTES) / stage_bytes + 1) : STAGES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x;            // which 128 output features (GATED: which `feat`)
    const int tile_m = blockIdx.y;            // which BN tokens
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(num_kb, kb_begin + kb_per_split);
    const int n_iters = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        // a fault recorded by an earlier CTA or kernel: do no work, so that a stuck
        // launch drains quickly instead of every CTA waiting out its own limit
        *abort_flag = (*(volatile int*)status != 0) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;

    pdl_trigger();
    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: TMA loads of the weight tile and the token tile.
            // The weights are written by no kernel, so the first ring of weight
            // tiles is fetched before waiting for the preceding kernel; the token
            // tiles (its output) follow after the wait.
            const int ahead = *abort_flag ? 0 : min(n_iters, n_stages);
            auto load_weights = [&](unsigned char* dst, uint64_t* bar, int k0) {
                // (packed weights: column 0 of the k-block's rows; row-major: column k0 of the matrix's rows)
                const int x = wp ? 0 : k0, y0 = wp ? (k0 / TC_BK) * wp : 0;
                if (GATED) {
                    tma_load_2d(dst, &map_w, bar, x, y0 + tile_n * feat);
                    tma_load_2d(dst + w_bytes / 2, &map_w, bar, x, y0 + gate_rows + tile_n * feat);
                } else {
                    tma_load_2d(dst, &map_w, bar, x, y0 + tile_n * TC_BM);
                }
            };
            for (int it = 0; it < ahead; ++it) {
                mbar_expect_tx(&full_bar[it], stage_bytes);
                load_weights(tiles + it * stage_bytes, &full_bar[it], (kb_begin + it) * TC_BK);
            }
            pdl_wait();
            for (int it = 0; it < ahead; ++it) {
                unsigned char* b_dst = tiles + it * stage_bytes + w_bytes;
                tma_load_2d(b_dst, &map_a, &full_bar[it], (kb_begin + it) * TC_BK, tile_m * BN);
            }
            int s = ahead % n_stages;
            uint32_t ph = (uint32_t)(ahead / n_stages) & 1u;
            for (int it = ahead; it < n_iters && !*abort_flag; ++it) {
                if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_EMPTY_WAIT); }
                    break;
                }
                unsigned char* a_dst = tiles + s * stage_bytes;
                mbar_expect_tx(&full_bar[s], stage_bytes);
                const int k0 = (kb_begin + it) * TC_BK;
                load_weights(a_dst, &full_bar[s], k0);
                tma_load_2d(a_dst + w_bytes, &map_a, &full_bar[s], k0, tile_m * BN);
                if (++s == n_stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            constexpr uint32_t idesc = instr_desc_bf16(TC_BM, BN);
            bool ok = !*abort_flag;
            int s = 0;
            uint32_t ph = 0;
            for (int it = 0; it < n_iters && ok; ++it) {
                if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_FULL_WAIT); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(tiles + s * stage_bytes);
                const uint32_t b_addr = a_addr + (uint32_t)w_bytes;
                const uint64_t adesc = smem_desc_sw128(a_addr);
                const uint64_t bdesc = smem_desc_sw128(b_addr);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k) {
                    // 16 bfloat16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
                    umma_bf16(tmem_acc, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                              (it > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);         // frees the stage once these MMAs have read it
                if (++s == n_stages) { s = 0; ph ^= 1u; }
            }
            if (ok) umma_commit(acc_bar);           // accumulator complete
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) ..
        const int quarter = warp & 3;
        bool ok = !*abort_flag;
        pdl_wait();                                   // C may still be read by the preceding kernel
        if (ok && n_iters > 0) {
            ok = mbar_wait(acc_bar, 0, abort_flag);
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_ACC_WAIT); }
        }
        tc_fence_after();
        if (GATED) {
            // Rows 0 .. feat-1 of the accumulator are gate features, the next `feat` the same features'
            // up values.  16 tokens at a time, every row's values (rounded to the activation type first,
            // as the unfused route stores them) go to shared memory (the ring is idle once the accumulator
            // is complete; two halves in turn, one barrier a round), and the threads share out the
            // 16 x feat results, a token's features side by side.
            // All four warps take the same decisions, so that the barrier below is always met.
            if (!ok) *abort_flag = 1;
            epilogue_sync();
            ok = !*abort_flag;
            const int row = quarter * 32 + lane;
            const int f0 = tile_n * feat;
            const uint32_t t_base = tmem_acc + ((uint32_t)(quarter * 32) << 16);
            const int t0 = tile_m * BN;
            float* xch = reinterpret_cast<float*>(tiles);            // [2][16 tokens][128 rows]
            const bool vec_ok = (((uintptr_t)C | (uintptr_t)(ldc * (long)sizeof(OutT))) & 15) == 0;
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (t0 + c >= M) break;                           // uniform over the four warps
                    uint32_t r[16];
                    tmem_ld16(t_base + (uint32_t)c, r);
                    tmem_ld_wait();
                    float* x = xch + ((c >> 4) & 1) * (16 * TC_BM);
                    if (row < 2 * feat) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            x[j * TC_BM + row] = to_f32<OutT>(from_f32<OutT>(__uint_as_float(r[j])));
                    }
                    epilogue_sync();
                    const int rows = min(16, M - (t0 + c));
                    // a thread finishes eight neighbouring features of one token and stores them as 16 bytes
                    // (feat is a multiple of 8, so 16 tokens x feat / 8 such pieces are at most one a thread)
                    const int pieces = feat >> 3;
                    const int t = row / pieces, f = (row - t * pieces) << 3;
                    if (t < rows && f0 + f < N) {
                        const float* xg = x + t * TC_BM + f;
                        OutT* dst = C + (long)(t0 + c + t) * ldc + f0 + f;
                        if (sizeof(OutT) == 2 && vec_ok && f0 + f + 8 <= N) {
                            const float4 g0 = *reinterpret_cast<const float4*>(xg), g1 = *reinterpret_cast<const float4*>(xg + 4);
                            const float4 u0 = *reinterpret_cast<const float4*>(xg + feat), u1 = *reinterpret_cast<const float4*>(xg + feat + 4);
                            const OutT v[8] = {from_f32<OutT>(gated_act(g0.x, u0.x)), from_f32<OutT>(gated_act(g0.y, u0.y)),
                                               from_f32<OutT>(gated_act(g0.z, u0.z)), from_f32<OutT>(gated_act(g0.w, u0.w)),
                                               from_f32<OutT>(gated_act(g1.x, u1.x)), from_f32<OutT>(gated_act(g1.y, u1.y)),
                                               from_f32<OutT>(gated_act(g1.z, u1.z)), from_f32<OutT>(gated_act(g1.w, u1.w))};
                            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
                        } else {
                            for (int j = 0; j < 8 && f0 + f + j < N; ++j)
                                dst[j] = from_f32<OutT>(gated_act(xg[j], xg[feat + j]));
                        }
                    }
                }
            }
        } else {
            // 16 tokens x 128 features at a time go through shared memory (the ring is idle once the
            // accumulator is complete; two halves in turn, one barrier a round) and leave as whole rows.
            // All four warps take the same decisions, so that the barrier below is always met.
            if (!ok) *abort_flag = 1;
            epilogue_sync();
            ok = !*abort_flag;
            const uint32_t t_base = tmem_acc + ((uint32_t)(quarter * 32) << 16);
            const int t0 = tile_m * BN;
            const int e = quarter * 32 + lane;                        // this thread's feature among the CTA's 128
            const int o0 = tile_n * TC_BM;
            const int cols = min(N - o0, TC_BM);
            float* slab = gridDim.z > 1 ? partial + (long)blockIdx.z * M * ld_partial : nullptr;
            const bool vec_ok = slab ? ((((uintptr_t)slab | (uintptr_t)(ld_partial * 4)) & 15) == 0)
                                     : ((((uintptr_t)C | (uintptr_t)(ldc * (long)sizeof(OutT))) & 15) == 0);
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (t0 + c >= M) break;                           // uniform over the four warps
                    uint32_t r[16];
                    if (n_iters > 0) {
                        tmem_ld16(t_base + (uint32_t)c, r);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = 0u;
                    }
                    unsigned char* half = tiles + ((c >> 4) & 1) * (16 * TC_BM * 4);
                    const int rows = min(16, M - (t0 + c));
                    if (slab) {
                        float* st = reinterpret_cast<float*>(half);
#pragma unroll
                        for (int j = 0; j < 16; ++j) st[j * TC_BM + e] = __uint_as_float(r[j]);
                        epilogue_sync();
                        tc_copy_rows<float, TC_BM, 16>(slab + (long)(t0 + c) * ld_partial + o0, ld_partial, st, rows,
                                                       cols, e, vec_ok);
                    } else {
                        OutT* st = reinterpret_cast<OutT*>(half);
#pragma unroll
                        for (int j = 0; j < 16; ++j) st[j * TC_BM + e] = from_f32<OutT>(__uint_as_float(r[j]));
                        epilogue_sync();
                        tc_copy_rows<OutT, TC_BM, 16>(C + (long)(t0 + c) * ldc + o0, ldc, st, rows, cols, e, vec_ok);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, TMEM_COLS);
    }
}

// ------------------------------------------------------------ tile order
// The order in which the persistent (CTA-pair) kernel walks over output tiles.  The CTAs
// (or CTA pairs) that run at the same time work on consecutive tiles, so these
// should share operands: token tiles go fastest inside panels of TC_RASTER_M
// token tiles, i.e. a weight tile is fetched from DRAM once per panel and used by
// up to TC_RASTER_M CTAs at about the same time out of L2, while the panel's
// activations (a few MB) stay in L2 throughout.  (With weight tiles fastest, the
// whole weight matrix, larger than L2, streamed from DRAM once per token tile.)
#define TC_RASTER_M 8
__device__ __forceinline__ void tc_raster(int tile, int tiles_n, int tiles_m, int& tn, int& tm) {
    const int per_panel = TC_RASTER_M * tiles_n;
    const int panel = tile / per_panel;
    const int within = tile - panel * per_panel;
    const int rows = min(TC_RASTER_M, tiles_m - panel * TC_RASTER_M);     // token tiles in this panel
    tn = within / rows;
    tm = panel * TC_RASTER_M + (within - tn * rows);
}

// ------------------------------------------------------------- pair variant
// For everything above 64 tokens: a persistent kernel (a loop over output tiles per
// CTA, the ring of shared-memory stages running on across tile boundaries, the
// accumulator double-buffered in tensor memory so that the epilogue of tile i
// overlaps the MMAs of tile i + 1) run by PAIRS of CTAs on neighbouring SMs
// (a cluster of two) that issue one MMA together (tcgen05 cta_group::2): a pair
// computes a 256 x 256 tile, each CTA holding 128 of the weight rows and 128 of
// the token rows in its shared memory and its own 128 x 256 half of the
// accumulator in its tensor memory.  Per 64-deep K step a CTA now fetches 32 KiB
// instead of 48 KiB for the same number of multiply-adds, which is what the
// one-CTA kernel runs out of (operand supply from L2), and the ring is 6 deep.
//   * both CTAs' producers load their halves; all four loads of a stage signal
//     the LEADER's full barrier (the even CTA), which the leader arms;
//   * the leader's MMA thread issues the MMAs and commits to BOTH CTAs' empty and
//     accumulator-full barriers (tcgen05.commit with a CTA mask);
//   * both CTAs' epilogue warps drain their own tensor memory and report to the
//     leader's accumulator-empty barrier.
// No load is multicast.  The two CTAs meet at a cluster barrier after set-up and
// before they leave, so neither touches the other's barriers outside its life.
// The token side of a pair's tile has room for BNT = 256, 128 or 64 tokens (each CTA holds half of it); a
// narrower tile leaves room for a deeper ring.  The tiles of a launch are `wt` <= BNT tokens wide, a
// multiple of 32 chosen by the launcher so that the token tiles are equally wide and a step of, say,
// 520 tokens is three tiles of 192 and not three of 256 (the box of the token rows' tensor map, the
// bytes a stage expects and the MMA's N all follow wt).  K may be split: a pair's units of work are (tile, K range) pairs, and with more than one
// split every unit writes its float partial sums to partial[split][token][feature] for the consumer
// (or the reduce kernel) to add, exactly as the one-tile kernel does.
template <int BNT>
struct Tc2 {
    static constexpr int W_BYTES = TC_BM * TC_BK * 2;              // 128 weight rows of a stage
    static constexpr int A_BYTES = (BNT / 2) * TC_BK * 2;          // this CTA's half of the token rows
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int STAGES = BNT == 256 ? 6 : (BNT == 128 ? 8 : 9);
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM = TILE_BYTES + 256 + 1024;        // + the epilogue's area below
};
#define TC2_XCH_BYTES (2 * 32 * 64 * 4)                      // GATED: two rounds of 32 tokens x 64 up values
#define TC2_GATED_OUT_BYTES (2 * 32 * 64 * 4)                // GATED: two rounds of 32 tokens x 64 results
#define TC2_OUT_BYTES (2 * 32 * 128 * 4)                     // two rounds of 32 tokens x 128 features on their way out

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* leader_bar, int x,
                                                 int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"((uint64_t)map), "r"(smem_u32(leader_bar) & TC2_PEER_MASK), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {      // arrives on this barrier in both CTAs
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {    // arrive on the even CTA's copy of `bar`
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & TC2_PEER_MASK) : "memory");
}

// ROPE: the q|k|v product of an attention layer with heads of 128, followed in the same kernel by what
// would otherwise be a kernel of its own (rope_kv.cu): a CTA's 128 features are exactly one head, so the
// epilogue, which has 32 tokens x 128 features of it in shared memory anyway, rotates a query head and
// writes it to C, rotates a key head straight into the tokens' slots of the paged cache, and copies a value
// head there.  The k and v columns never go to memory as activations (a third of what the rotary kernel
// read and wrote).  Values are rounded to bfloat16 before the rotation, as the separate kernel finds them,
// and rotated by the same expressions.
struct TcRope {
    const int* positions;       // [tokens] absolute position
    const int* slots;           // [tokens] page * page_size + offset, < 0: no cache write for the token
    const float* cos_table;     // [positions, 64]
    const float* sin_table;
    bf16* k_cache;              // the layer's keys: [page][kv head][page_size][128], pages page_stride elements apart
    bf16* v_cache;
    long page_stride;
    int page_size, n_heads, n_kv_heads;
};
// How the 128 epilogue threads share a round of 32 tokens x 128 features: four threads a token row, thread
// q of a row owning the pairs (j, j + 64) for j in [16 q, 16 q + 16).  What a thread needs from global memory for
// a round (its token's position and slot, then 16 cosines and sines) is asked for well before it is used: the
// position and slot a round ahead, the table values before the round's accumulator is read from tensor memory.
#define TC_ROPE_PITCH 136                                   // staging row pitch in elements: rows 272 bytes apart spread over the banks
struct TcRopeRow {
    int pos, slot;
    float4 c[4], s[4];
};
__device__ __forceinline__ void tc_rope_ask_row(const TcRope& rp, TcRopeRow& w, int t, bool real) {
    w.pos = real ? rp.positions[t] : 0;
    w.slot = real ? rp.slots[t] : -1;
}
__device__ __forceinline__ void tc_rope_ask_table(const TcRope& rp, TcRopeRow& w, int q, bool rotates) {
    if (!rotates) return;
    const float4* cs = reinterpret_cast<const float4*>(rp.cos_table + (long)w.pos * 64 + 16 * q);
    const float4* sn = reinterpret_cast<const float4*>(rp.sin_table + (long)w.pos * 64 + 16 * q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w.c[i] = cs[i];
        w.s[i] = sn[i];
    }
}
// one token row of one head from the staging area `x` (128 values): a query head is rotated and goes to C, a
// key head is rotated into the token's cache slot, a value head is copied there
__device__ __forceinline__ void tc_rope_row(const TcRope& rp, const TcRopeRow& w, bf16* __restrict__ C, long ldc,
                                            const bf16* __restrict__ x, int t, int o0, int q) {
    constexpr int HD = 128, HALF = 64;
    const int head = o0 / HD;
    const bool is_query = head < rp.n_heads, is_key = head < rp.n_heads + rp.n_kv_heads;
    bf16* dst;
    if (is_query) {
        dst = C + (long)t * ldc + o0;
    } else {
        if (w.slot < 0) return;
        const long page = w.slot / rp.page_size;
        const int off = w.slot - (int)page * rp.page_size;
        const int kvh = head - rp.n_heads - (is_key ? 0 : rp.n_kv_heads);
        dst = (is_key ? rp.k_cache : rp.v_cache) + page * rp.page_stride + (long)kvh * rp.page_size * HD + (long)off * HD;
        if (!is_key) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(dst + 32 * q + 8 * i) = *reinterpret_cast<const uint4*>(x + 32 * q + 8 * i);
            return;
        }
    }
    const int j = 16 * q;
#pragma unroll
    for (int v = 0; v < 2; ++v) {                           // two vectors of eight pairs
        const uint4 a = *reinterpret_cast<const uint4*>(x + j + 8 * v);
        const uint4 b = *reinterpret_cast<const uint4*>(x + j + 8 * v + HALF);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        const float c[8] = {w.c[2 * v].x, w.c[2 * v].y, w.c[2 * v].z, w.c[2 * v].w,
                            w.c[2 * v + 1].x, w.c[2 * v + 1].y, w.c[2 * v + 1].z, w.c[2 * v + 1].w};
        const float sv[8] = {w.s[2 * v].x, w.s[2 * v].y, w.s[2 * v].z, w.s[2 * v].w,
                             w.s[2 * v + 1].x, w.s[2 * v + 1].y, w.s[2 * v + 1].z, w.s[2 * v + 1].w};
        uint4 lo, hi;
        __nv_bfloat162* lp = reinterpret_cast<__nv_bfloat162*>(&lo);
        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x1 = __bfloat1622float2(ap[i]), x2 = __bfloat1622float2(bp[i]);
            lp[i] = __floats2bfloat162_rn(x1.x * c[2 * i] - x2.x * sv[2 * i], x1.y * c[2 * i + 1] - x2.y * sv[2 * i + 1]);
            hp[i] = __floats2bfloat162_rn(x2.x * c[2 * i] + x1.x * sv[2 * i], x2.y * c[2 * i + 1] + x1.y * sv[2 * i + 1]);
        }
        *reinterpret_cast<uint4*>(dst + j + 8 * v) = lo;
        *reinterpret_cast<uint4*>(dst + j + 8 * v + HALF) = hi;
    }
}

// GATED as in gemm_tc_kernel: each CTA's 128 weight rows are 64 gate rows and the 64 up rows of the
// same features, a pair's tile is 128 features wide, and the epilogue writes silu(gate) * up
// (whole K only: `splits` is 1 then).
template <int BNT, typename OutT, bool GATED, bool ROPE>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_pair_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
    OutT* __restrict__ C, long ldc, int M, int N, int K, int tiles_n, int num_tiles,
    int* __restrict__ status, int gate_rows, int splits, int kb_per_split, float* __restrict__ partial,
    long ld_partial, const TcRope rope, int wp, int wt) {
    using L = Tc2<BNT>;
    static_assert(!GATED || BNT == 256, "the gated epilogue is written for 256-token tiles");
    static_assert(!ROPE || (!GATED && sizeof(OutT) == 2), "the rotary epilogue writes bfloat16 and is not gated");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(tiles + L::TILE_BYTES);
    uint64_t* empty_bar = full_bar + L::STAGES;
    uint64_t* acc_full = empty_bar + L::STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(tiles + L::TILE_BYTES + 256);      // GATED only
    unsigned char* staged = tiles + L::TILE_BYTES + 256;                      // plain epilogue only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                   // 0: leader
    const int pair = (int)blockIdx.x >> 1, num_pairs = (int)gridDim.x >> 1;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int num_units = num_tiles * splits;
    const int my_units = (pair < num_units) ? (num_units - 1 - pair) / num_pairs + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L::STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);                    // four epilogue warps in each of the two CTAs
        }
        *abort_flag = (*(volatile int*)status != 0) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                     // both CTAs' barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // This kernel neither starts before its predecessor has finished nor lets its successor in early
    // (no programmatic launch attribute, no pdl_trigger): with either, runs in which a CTA pair shared
    // the GPU with another kernel that also allocates tensor memory stalled for good now and then.

    // unit i of this pair: its tile (tn: features, tm: tokens), its split and that split's k-blocks
    auto unit = [&](int i, int& tn, int& tm, int& split, int& kb0, int& kb1) {
        const int u = pair + i * num_pairs;
        split = u / num_tiles;
        tc_raster(u - split * num_tiles, tiles_n, num_tiles / tiles_n, tn, tm);
        kb0 = split * kb_per_split;
        kb1 = min(num_kb, kb0 + kb_per_split);
    };

    // this CTA's 128 weight rows of a stage (GATED: 64 gate rows and the 64 up rows of the same features)
    auto load_weights = [&](unsigned char* dst, uint64_t* bar, int kb, int tn) {
        const int x = wp ? 0 : kb * TC_BK, y0 = wp ? kb * wp : 0;         // (packed weights: see the file's head)
        if (GATED) {
            const int f0 = tn * 128 + (int)rank * 64;
            tma_load_2d_pair(dst, &map_w, bar, x, y0 + f0);
            tma_load_2d_pair(dst + L::W_BYTES / 2, &map_w, bar, x, y0 + gate_rows + f0);
        } else {
            tma_load_2d_pair(dst, &map_w, bar, x, y0 + tn * 256 + (int)rank * TC_BM);
        }
    };

    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            // ---- producer (both CTAs): this CTA's 128 weight rows and BNT/2 token rows of each stage,
            // unit after unit, k-block after k-block, through the ring
            pdl_wait();
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int i = 0; i < my_units && ok; ++i) {
                int tn, tm, split, kb0, kb1;
                unit(i, tn, tm, split, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_EMPTY_WAIT); }
                        ok = false;
                        break;
                    }
                    unsigned char* dst = tiles + s * L::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * (L::W_BYTES + (wt / 2) * TC_BK * 2));
                    load_weights(dst, &full_bar[s], kb, tn);
                    tma_load_2d_pair(dst + L::W_BYTES, &map_a, &full_bar[s], kb * TC_BK,
                                     tm * wt + (int)rank * (wt / 2));
                    if (++s == L::STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (leader only): one 256 x wt x 16 MMA per 16 columns of K, for both CTAs
            const uint32_t idesc = instr_desc_bf16(256, wt);
            int s = 0;
            uint32_t ph = 0;
            bool ok = !*abort_flag;
            for (int i = 0; i < my_units && ok; ++i) {
                int tn, tm, split, kb0, kb1;
                unit(i, tn, tm, split, kb0, kb1);
                const int buf = i & 1;
                const uint32_t use = (uint32_t)(i >> 1);
                if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_ACC_WAIT); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * 256);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_FULL_WAIT); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t w_addr = smem_u32(tiles + s * L::STAGE_BYTES);
                    const uint64_t adesc = smem_desc_sw128(w_addr);
                    const uint64_t bdesc = smem_desc_sw128(w_addr + L::W_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(tmem_acc, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                       (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[s]);
                    if (++s == L::STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue warps 2..5 of both CTAs: this CTA's 128 output features of the pair's tile
        const int quarter = warp & 3;
        bool ok = true;
        uint32_t rounds_out = 0;                            // 32-token rounds written so far: picks the staging half
        pdl_wait();
        for (int i = 0; i < my_units && ok; ++i) {
            const int buf = i & 1;
            const uint32_t use = (uint32_t)(i >> 1);
            bool got = mbar_wait(&acc_full[buf], use & 1u, abort_flag);
            if (!got && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, TC_ERR_ACC_WAIT); }
            epilogue_sync();                                // the four warps decide together (they share barriers below)
            got = !*abort_flag;
            if (!got) {
                ok = false;
                break;
            }
            tc_fence_after();
            int tn, tm, split, kb0, kb1;
            unit(i, tn, tm, split, kb0, kb1);
            const int t0 = tm * wt;
            const uint32_t t_base = tmem_base + (uint32_t)(buf * 256) + ((uint32_t)(quarter * 32) << 16);
            if (GATED) {
                // accumulator lanes 0..63: gate features, 64..127: the same features' up values; the
                // gate warps finish the even tokens, the up warps the odd ones, trading the values
                // the other side needs through shared memory, 32 tokens at a time
                const bool is_up = quarter >= 2;
                const int col = (quarter & 1) * 32 + lane;
                const int f0 = tn * 128 + (int)rank * 64;   // first of this CTA's 64 features
                const bool vec_ok = (((uintptr_t)C | (uintptr_t)(ldc * (long)sizeof(OutT))) & 15) == 0;
#pragma unroll 1
                for (int c = 0; c < wt; c += 32) {
                    if (t0 + c >= M) break;                 // uniform over the four warps
                    uint32_t r[32];
                    tmem_ld16(t_base + (uint32_t)c, r);
                    tmem_ld16(t_base + (uint32_t)c + 16u, r + 16);
                    tmem_ld_wait();
                    const uint32_t half = rounds_out++ & 1u;
                    float* x = xch + half * (32 * 64);
                    OutT* st = reinterpret_cast<OutT*>(staged + TC2_XCH_BYTES) + half * (32 * 64);
                    const int mine = is_up ? 1 : 0;         // parity of the tokens this warp finishes
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if ((j & 1) != mine)
                            x[j * 64 + col] = to_f32<OutT>(from_f32<OutT>(__uint_as_float(r[j])));
                    epilogue_sync();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if ((j & 1) != mine) continue;
                        const float own = to_f32<OutT>(from_f32<OutT>(__uint_as_float(r[j])));
                        const float other = x[j * 64 + col];
                        st[j * 64 + col] = from_f32<OutT>(is_up ? gated_act(other, own) : gated_act(own, other));
                    }
                    epilogue_sync();                        // the 32 x 64 results leave as whole rows
                    if (f0 < N)
                        tc_copy_rows<OutT, 64>(C + (long)(t0 + c) * ldc + f0, ldc, st, min(32, M - (t0 + c)),
                                               min(N - f0, 64), quarter * 32 + lane, vec_ok);
                }
            } else {
                // each thread holds one feature's values of 32 tokens at a time: they go through shared memory
                // ([token][feature], alternating halves so that one barrier per round is enough) and leave as
                // whole rows
                const int e = quarter * 32 + lane;              // this thread's feature among the CTA's 128
                const int o0 = tn * 256 + (int)rank * TC_BM;
                const int cols = N - o0;                        // features of this CTA that exist (may be <= 0)
                float* slab = splits > 1 ? partial + (long)split * M * ld_partial : nullptr;
                const bool vec_ok = slab ? ((((uintptr_t)slab | (uintptr_t)(ld_partial * 4)) & 15) == 0)
                                         : ((((uintptr_t)C | (uintptr_t)(ldc * (long)sizeof(OutT))) & 15) == 0);
                if constexpr (ROPE) {
                    // (ROPE: whole K, bfloat16, one head a CTA; see TcRope)
                    const int row = e >> 2, q4 = e & 3;         // this thread's token row of a round and its quarter of the pairs
                    const bool rotates = o0 / 128 < rope.n_heads + rope.n_kv_heads;
                    TcRopeRow cur, nxt;
                    tc_rope_ask_row(rope, cur, t0 + row, t0 + row < M);
#pragma unroll 1
                    for (int c = 0; c < wt; c += 32) {
                        if (t0 + c >= M) break;                 // uniform over the four warps
                        const int t = t0 + c + row;
                        tc_rope_ask_table(rope, cur, q4, rotates && t < M);
                        tc_rope_ask_row(rope, nxt, t + 32, c + 32 < wt && t + 32 < M);
                        uint32_t r[32];
                        tmem_ld16(t_base + (uint32_t)c, r);
                        tmem_ld16(t_base + (uint32_t)c + 16u, r + 16);
                        tmem_ld_wait();
                        bf16* st = reinterpret_cast<bf16*>(staged + (rounds_out++ & 1u) * (TC2_OUT_BYTES / 2));
#pragma unroll
                        for (int j = 0; j < 32; ++j) st[j * TC_ROPE_PITCH + e] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        epilogue_sync();
                        if (cols > 0 && t < M)
                            tc_rope_row(rope, cur, reinterpret_cast<bf16*>(C), ldc, st + row * TC_ROPE_PITCH, t, o0, q4);
                        cur.pos = nxt.pos;
                        cur.slot = nxt.slot;
                    }
                } else {
#pragma unroll 1
                for (int c = 0; c < wt; c += 32) {
                    if (t0 + c >= M) break;                     // uniform over the four warps
                    uint32_t r[32];
                    tmem_ld16(t_base + (uint32_t)c, r);
                    tmem_ld16(t_base + (uint32_t)c + 16u, r + 16);
                    tmem_ld_wait();
                    unsigned char* half = staged + (rounds_out++ & 1u) * (TC2_OUT_BYTES / 2);
                    const int rows = min(32, M - (t0 + c));
                    if (slab) {
                        float* st = reinterpret_cast<float*>(half);
#pragma unroll
                        for (int j = 0; j < 32; ++j) st[j * 128 + e] = __uint_as_float(r[j]);
                        epilogue_sync();
                        if (cols > 0)
                            tc_copy_rows<float, 128>(slab + (long)(t0 + c) * ld_partial + o0, ld_partial, st, rows,
                                                     min(cols, 128), e, vec_ok);
                    } else {
                        OutT* st = reinterpret_cast<OutT*>(half);
#pragma unroll
                        for (int j = 0; j < 32; ++j) st[j * 128 + e] = from_f32<OutT>(__uint_as_float(r[j]));
                        epilogue_sync();
                        if (cols > 0)
                            tc_copy_rows<OutT, 128>(C + (long)(t0 + c) * ldc + o0, ldc, st, rows, min(cols, 128), e,
                                                    vec_ok);
                    }
                }
            }
                }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                     // the peer is done with this CTA's barriers and memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    // Neither CTA leaves before both have given their tensor memory back.  Without this barrier a CTA of the
    // next kernel could take the SM of the CTA that left first and allocate tensor memory there while the
    // peer's paired deallocation was still to come; such runs stalled for good now and then.
    cluster_sync_all();
}

// Width in tokens of the pair kernel's tiles for M tokens and room for `bnt`: as many tiles as whole ones
// would take, equally wide, a multiple of 32 (the epilogue's round).  Each CTA's box of token rows is half of it.
static int tc_pair_tile_tokens(int M, int bnt) {
    const int tiles = (M + bnt - 1) / bnt;
    const int wt = ((M + tiles - 1) / tiles + 31) / 32 * 32;
    return wt < bnt ? wt : bnt;
}

template <int BNT, typename OutT, bool GATED = false, bool ROPE = false>
static int launch_tc_pair(const CUtensorMap& map_w, const CUtensorMap& map_a, void* C, long ldc, int M, int N,
                          int K, int num_sms, int* status, cudaStream_t stream, int gate_rows = 0, int splits = 1,
                          int kb_per_split = 0, float* partial = nullptr, long ld_partial = 0,
                          const TcRope* rope_args = nullptr, int wp = 0) {
    static bool configured = false;
    auto kernel = gemm_tc_pair_kernel<BNT, OutT, GATED, ROPE>;
    TcRope rope = {};
    if (rope_args) rope = *rope_args;
    constexpr int smem = Tc2<BNT>::SMEM + (GATED ? TC2_XCH_BYTES + TC2_GATED_OUT_BYTES : TC2_OUT_BYTES);
    static_assert(smem <= 232448, "more shared memory than a CTA can have");
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles_n = GATED ? (N + 127) / 128 : (N + 255) / 256;
    const int wt = tc_pair_tile_tokens(M, BNT);
    const int num_tiles = tiles_n * ((M + wt - 1) / wt);
    const long num_units = (long)num_tiles * splits;
    const int pairs = num_units < num_sms / 2 ? (int)num_units : num_sms / 2;
    if (splits == 1) kb_per_split = (K + TC_BK - 1) / TC_BK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    // Launched in plain stream order (no programmatic overlap with its neighbours): see the note in the kernel.
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, map_w, map_a, (OutT*)C, ldc, M, N, K, tiles_n, num_tiles, status,
                                   gate_rows, splits, kb_per_split, partial, ld_partial, rope, wp, wt);
}

template <typename OutT>
static int dispatch_tc_pair(int bnt, const CUtensorMap& map_w, const CUtensorMap& map_a, void* C, long ldc, int M,
                            int N, int K, int num_sms, int* status, cudaStream_t stream, int splits,
                            int kb_per_split, float* partial, long ld_partial, int wp) {
    switch (bnt) {
        case 64: return launch_tc_pair<64, OutT>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, splits, kb_per_split, partial, ld_partial, nullptr, wp);
        case 128: return launch_tc_pair<128, OutT>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, splits, kb_per_split, partial, ld_partial, nullptr, wp);
        case 256: return launch_tc_pair<256, OutT>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, splits, kb_per_split, partial, ld_partial, nullptr, wp);
    }
    return (int)cudaErrorInvalidValue;
}

// C[t, o] = sum over splits of partial[z][t][o], added in the order z = 0, 1, ...
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, long ld_partial, int splits,
                                     OutT* __restrict__ C, long ldc, int M, int N) {
    pdl_wait();
    pdl_trigger();
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (o >= N) return;
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) acc += partial[((long)z * M + t) * ld_partial + o];
    C[(long)t * ldc + o] = from_f32<OutT>(acc);
}

// C = the sum of `splits` slabs partial[z][M][ld_partial] (what fl_gemm_tc_partial leaves), for a
// consumer that has no kernel of its own that adds the slabs while it reads them.
FL_API int fl_splitk_reduce(const float* partial, long ld_partial, int splits, void* C, int c_dtype, long ldc,
                            int M, int N, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (splits < 1 || M > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + 255) / 256, M);
    if (c_dtype == FL_BF16)
        return fl_launch(splitk_reduce_kernel<bf16>, grid, dim3(256), 0, stream, partial, ld_partial, splits,
                         (bf16*)C, ldc, M, N);
    if (c_dtype == FL_F32)
        return fl_launch(splitk_reduce_kernel<float>, grid, dim3(256), 0, stream, partial, ld_partial, splits,
                         (float*)C, ldc, M, N);
    return (int)cudaErrorInvalidValue;
}

// dst[kb][n][c] = src[n][kb * 64 + c] (zero where kb * 64 + c >= K): a weight matrix packed by k-block, so that
// the 128 rows x 64 columns which a stage loads lie in one piece of memory.  One thread moves 16 bytes.
__global__ void pack_weight_kernel(const bf16* __restrict__ src, long ld, bf16* __restrict__ dst, long N, int K,
                                   int num_kb) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;       // over num_kb * N * 8 pieces of 8 values
    if (i >= (long)num_kb * N * 8) return;
    const int piece = (int)(i & 7);
    const long n = (i >> 3) % N, kb = (i >> 3) / N;
    const int k = (int)kb * TC_BK + piece * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    const bf16* s = src + n * ld + k;
    if (k + 8 <= K && ((((uintptr_t)s) & 15) == 0)) {
        v = *reinterpret_cast<const uint4*>(s);
    } else {
        bf16* e = reinterpret_cast<bf16*>(&v);
        for (int c = 0; c < 8 && k + c < K; ++c) e[c] = s[c];
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = v;
}

// Packs W[N, K] (bfloat16, `ld` elements between rows) into dst[ceil(K / 64)][N][64] for the kernels above.
FL_API int fl_pack_weight(const void* W, long ld, void* dst, long N, int K, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return 0;
    if (((uintptr_t)dst) & 15) return (int)cudaErrorMisalignedAddress;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const long pieces = (long)num_kb * N * 8;
    pack_weight_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, stream>>>((const bf16*)W, ld, (bf16*)dst, N, K, num_kb);
    return fl_launch_status();
}

// ----------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, cols] bfloat16 matrix with `ld` elements between rows, read in boxes
// of box_rows x 64 elements with the 128-byte swizzle; out-of-range reads give zeros.
static int make_map(CUtensorMap* map, const void* base, long rows, long cols, long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    if (((uintptr_t)base & 15) || ((ld * 2) & 15)) return (int)cudaErrorMisalignedAddress;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                    box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// The tensor map of a weight matrix [rows, K] in either layout: row-major with `ldw` elements between rows, or,
// with ldw == 0, packed by k-block ([ceil(K / 64)][rows][64]: a matrix of 64 columns whose k-blocks follow one
// another; a tile that ends beyond a k-block's rows reads on into the next one, or into nothing past the end,
// and what it reads there lands in accumulator rows that no epilogue stores).
static int make_w_map(CUtensorMap* map, const void* W, long rows, long K, long ldw, int box_rows) {
    if (ldw == 0) return make_map(map, W, rows * ((K + TC_BK - 1) / TC_BK), TC_BK, TC_BK, box_rows);
    return make_map(map, W, rows, K, ldw, box_rows);
}

template <int BN, int STAGES, typename OutT, bool GATED = false>
static int launch_tc(const CUtensorMap& map_w, const CUtensorMap& map_a, void* C, long ldc,
                     float* partial, long ld_partial, int M, int N, int K, int splits,
                     int kb_per_split, int* status, cudaStream_t stream, int gate_rows = 0, int feat = 64, int wp = 0) {
    using L = TcSmem<BN, STAGES>;
    // This kernel is launched with programmatic overlap, so CTAs of it and of its neighbours in the stream share
    // SMs; as many of them as fit an SM by shared memory must find their tensor-memory columns free at once, or an
    // allocation would wait for a CTA that waits for its predecessor (see fl_launch).  Every kernel launched that
    // way which takes tensor memory is an instance of this one, and the instance with the least shared memory
    // decides how many fit.
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int SMALLEST_TOTAL = 96 * 1024;                  // no instance has less shared memory than this ...
    constexpr int MOST_COLS = 256;                             // ... and none takes more columns than this
    static_assert(L::TOTAL >= SMALLEST_TOTAL && TMEM_COLS <= MOST_COLS, "a new instance: revise the two bounds");
    static_assert(TMEM_COLS + (232448 - L::TOTAL) / SMALLEST_TOTAL * MOST_COLS <= 512,
                  "CTAs that fit an SM together could ask for more than its 512 tensor-memory columns");
    static bool configured = false;
    auto kernel = gemm_tc_kernel<BN, STAGES, OutT, GATED>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(GATED ? (N + feat - 1) / feat : (N + TC_BM - 1) / TC_BM, (M + BN - 1) / BN, splits);
    return fl_launch(kernel, grid, dim3(TC_THREADS), (size_t)L::TOTAL, stream, map_w, map_a, (OutT*)C, ldc,
                     partial, ld_partial, M, N, K, kb_per_split, status, gate_rows, feat, wp);
}

template <typename OutT>
static int dispatch_tc(int bn, const CUtensorMap& map_w, const CUtensorMap& map_a, void* C, long ldc,
                       float* partial, long ld_partial, int M, int N, int K, int splits,
                       int kb_per_split, int* status, cudaStream_t stream, int wp) {
    switch (bn) {
        case 16: return launch_tc<16, 6, OutT>(map_w, map_a, C, ldc, partial, ld_partial, M, N, K, splits, kb_per_split, status, stream, 0, 64, wp);
        case 32: return launch_tc<32, 5, OutT>(map_w, map_a, C, ldc, partial, ld_partial, M, N, K, splits, kb_per_split, status, stream, 0, 64, wp);
        case 64: return launch_tc<64, 4, OutT>(map_w, map_a, C, ldc, partial, ld_partial, M, N, K, splits, kb_per_split, status, stream, 0, 64, wp);
        case 128: return launch_tc<128, 3, OutT>(map_w, map_a, C, ldc, partial, ld_partial, M, N, K, splits, kb_per_split, status, stream, 0, 64, wp);
        case 256: return launch_tc<256, 4, OutT>(map_w, map_a, C, ldc, partial, ld_partial, M, N, K, splits, kb_per_split, status, stream, 0, 64, wp);
    }
    return (int)cudaErrorInvalidValue;
}

// Token-tile width and K splits of the one-tile kernel for a problem: the smallest
// tile that holds the tokens (up to 256), and as many splits as it takes to give
// every SM a CTA or two.  Products of more than 128 tokens that need no split go to
// the CTA-pair kernel, reported as width 512.
static void plan_one_tile(int M, int N, int K, int num_sms, int* bn_out, int* splits_out) {
    int bn = 16;
    while (bn < 256 && bn < M) bn *= 2;
    const int tiles = ((N + TC_BM - 1) / TC_BM) * ((M + bn - 1) / bn);
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    // CTAs that can be resident at once: two per SM for token tiles up to 128
    // wide (their ring of stages is sized for that), one for 256.  Splitting K so
    // that all CTAs fit in one wave keeps every SM streaming until the end.
    const int target = bn <= 128 ? 2 * num_sms : num_sms;
    int splits = 1;
    if (tiles < target) {
        splits = target / tiles;
        const int most = num_kb / 4 > 0 ? num_kb / 4 : 1;       // at least 4 k-blocks per split
        if (splits > most) splits = most;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    const int per = (num_kb + splits - 1) / splits;
    splits = (num_kb + per - 1) / per;                          // no empty split
    if (bn == 256 && splits == 1 && num_sms >= 2) bn = 512;     // 512 stands for the CTA-pair kernel (256 x 256 tiles)
    *bn_out = bn;
    *splits_out = splits;
}

// Modelled microseconds of a product [M, K] x [N, K]^T run as (bn, splits): bn 64, 128, 256: the one-tile
// kernel with that token tile; 512, 640: the CTA-pair kernel, 256 or 128 tokens wide.  `deferred`: the
// partial sums of a split K are left to the consumer kernel, which adds them as it reads them; else a reduce
// kernel follows.  The constants were fitted (least squares on the logarithm) to event-timed runs of every
// candidate on B200 for 12 weight shapes of 2048 to 102400 features and 2048 to 22016 inputs at 80 to 768
// tokens: 8 % root-mean-square error, and the candidate the model picks is within 1.6 % of the best one on
// average (15 % at worst).  One-tile CTAs cost a fixed start plus a time per 64-deep K step that is a fifth
// shorter when a CTA has its SM to itself; a pair costs a fixed 7.3 us a launch and 0.28 to 0.31 us a K step;
// no product is faster than its operands stream from memory; partial sums cost their bytes.
static double tc_cost(int M, int N, int K, int num_sms, int bn, int splits, int deferred) {
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int per = (num_kb + splits - 1) / splits;
    double t;
    if (bn >= 512) {
        const int bnt = bn == 512 ? 256 : bn - 512;
        const long units = (long)((N + 255) / 256) * ((M + bnt - 1) / bnt) * splits;
        const long pairs = num_sms / 2;
        const long rounds = (units + pairs - 1) / pairs;
        t = 7.29 + (double)rounds * per * (bnt == 256 ? 0.312 : 0.283);
    } else {
        const long ctas = (long)((N + TC_BM - 1) / TC_BM) * ((M + bn - 1) / bn) * splits;
        const long slots = (bn <= 128 ? 2L : 1L) * num_sms;
        const long rounds = (ctas + slots - 1) / slots;
        const double start = bn == 64 ? 2.11 : (bn == 128 ? 1.95 : 4.11);
        const double step = bn == 64 ? 0.374 : (bn == 128 ? 0.481 : 0.398);
        double load = 1.0;
        if (bn <= 128) {
            const double per_sm = (double)ctas / rounds / num_sms;    // CTAs on an SM in a round
            if (per_sm <= 1.0) load = 0.80 + 0.20 * per_sm;
        }
        t = (double)rounds * (start + per * step * load);
    }
    const double stream = ((double)N * K + (double)M * K) * 2.0 / 6.01e6 + 3.0;
    if (t < stream) t = stream;
    if (splits > 1) {
        const double slab_mb = (double)splits * M * N * 4.0 / 1.0e6;
        t += deferred ? slab_mb / 3.88 : 1.31 + slab_mb / 1.70;
    }
    return t;
}

// The plan for a product: up to 64 tokens the one-tile kernel (it overlaps with its neighbours in the
// stream, which counts most for the short kernels of a decode step), with the smallest tile that holds
// the tokens and K split until every SM has a CTA or two; above 64 tokens the cheapest candidate by
// tc_cost: the one-tile kernel with 64-, 128- or 256-token tiles (up to 1024 tokens; it has four times
// the CTAs of the pair kernel, which small weight matrices need) or the CTA-pair kernel (reported as 512:
// 256 tokens wide, or 640: 128 wide, for at most 128 tokens), each with 1 to 16 K splits of at least four
// k-blocks.  Of equally cheap candidates the one with fewer splits wins.
FL_API void fl_gemm_tc_plan_for(int M, int N, int K, int num_sms, int deferred, int* bn_out, int* splits_out) {
    if (M <= 64 || num_sms < 2) {
        plan_one_tile(M, N, K, num_sms, bn_out, splits_out);
        return;
    }
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int widths[4] = {M <= 128 ? 640 : 512, 64, 128, 256};
    int best_bn = widths[0], best_sp = 1;
    double best_cost = -1.0;
    for (int w = 0; w < 4; ++w) {
        const int bn = widths[w];
        if (bn < 512 && (M > 1024 || (bn == 64 && M > 256))) continue;
        for (int sp = 1; sp <= 16; ++sp) {
            const int per = (num_kb + sp - 1) / sp;
            if ((num_kb + per - 1) / per != sp) continue;           // no empty split
            if (sp > 1 && per < 4) break;
            const double cost = tc_cost(M, N, K, num_sms, bn, sp, deferred);
            if (best_cost < 0.0 || cost < best_cost * 0.99) {
                best_cost = cost;
                best_bn = bn;
                best_sp = sp;
            }
        }
    }
    *bn_out = best_bn;
    *splits_out = best_sp;
}

FL_API void fl_gemm_tc_plan(int M, int N, int K, int num_sms, int* bn_out, int* splits_out) {
    fl_gemm_tc_plan_for(M, N, K, num_sms, 0, bn_out, splits_out);
}

// A: [M, K] bfloat16 with lda elements between rows; W: [N, K] bfloat16 with ldw, or packed by k-block
// (fl_pack_weight) with ldw == 0;
// C: [M, N] bfloat16 or float with ldc.  lda and ldw must be multiples of 8 and
// the bases 16-byte aligned (what a TMA descriptor wants).  `workspace` holds
// splits * M * round_up(N, 4) floats when the plan splits K (bn and splits come
// from fl_gemm_tc_plan, or 0 to plan here).
static int gemm_tc_impl(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc,
                        int M, int N, int K, int bn, int splits, float* workspace, long workspace_floats,
                        int num_sms, int* status, cudaStream_t stream, int skip_reduce) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    if (bn == 0) fl_gemm_tc_plan_for(M, N, K, num_sms, skip_reduce, &bn, &splits);
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > num_kb) return (int)cudaErrorInvalidValue;
    const int kb_per_split = (num_kb + splits - 1) / splits;
    if ((long)(splits - 1) * kb_per_split >= num_kb) return (int)cudaErrorInvalidValue;
    const long ld_partial = ((long)N + 3) / 4 * 4;
    if (splits > 1 && (workspace == nullptr || workspace_floats < (long)splits * M * ld_partial))
        return (int)cudaErrorMemoryAllocation;
    if (bn <= 256 && (M + bn - 1) / bn > 65535) return (int)cudaErrorInvalidValue;
    CUtensorMap map_w, map_a;
    int rc = make_w_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc) return rc;
    const int wp = ldw == 0 ? N : 0;
    const bool paired = bn >= 512;                           // 512, 640, 576: pair kernel, 256 / 128 / 64 tokens wide
    const int bnt = bn == 512 ? 256 : bn - 512;
    if (paired && (num_sms < 2 || (bnt != 64 && bnt != 128 && bnt != 256))) return (int)cudaErrorInvalidValue;
    rc = make_map(&map_a, A, M, K, lda, paired ? tc_pair_tile_tokens(M, bnt) / 2 : bn);
    if (rc) return rc;
    if (paired) {                                            // each CTA of a pair loads half of the token rows
        float* part = splits > 1 ? workspace : nullptr;
        if (c_dtype == FL_BF16)
            rc = dispatch_tc_pair<bf16>(bnt, map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, splits, kb_per_split, part, ld_partial, wp);
        else if (c_dtype == FL_F32)
            rc = dispatch_tc_pair<float>(bnt, map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, splits, kb_per_split, part, ld_partial, wp);
        else
            return (int)cudaErrorInvalidValue;
    } else if (c_dtype == FL_BF16) {
        rc = dispatch_tc<bf16>(bn, map_w, map_a, C, ldc, workspace, ld_partial, M, N, K, splits, kb_per_split, status, stream, wp);
    } else if (c_dtype == FL_F32) {
        rc = dispatch_tc<float>(bn, map_w, map_a, C, ldc, workspace, ld_partial, M, N, K, splits, kb_per_split, status, stream, wp);
    } else {
        return (int)cudaErrorInvalidValue;
    }
    if (rc || splits == 1 || skip_reduce) return rc;
    return fl_splitk_reduce(workspace, ld_partial, splits, C, c_dtype, ldc, M, N, stream);
}

FL_API int fl_gemm_tc(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc,
                      int M, int N, int K, int bn, int splits, float* workspace, long workspace_floats,
                      int num_sms, int* status, cudaStream_t stream) {
    return gemm_tc_impl(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, bn, splits, workspace, workspace_floats,
                        num_sms, status, stream, 0);
}

// The same, but with splits > 1 the partial sums stay in the workspace
// ([splits][M][round_up(N, 4)] floats) for a consumer kernel that adds them as
// it reads; C is not written then.
FL_API int fl_gemm_tc_partial(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype,
                              long ldc, int M, int N, int K, int bn, int splits, float* workspace,
                              long workspace_floats, int num_sms, int* status, cudaStream_t stream) {
    return gemm_tc_impl(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, bn, splits, workspace, workspace_floats,
                        num_sms, status, stream, 1);
}

// The SwiGLU feed-forward's first product with its activation: W holds the gate matrix [I, K] and
// below it the up matrix [I, K]; C[M, I] = silu(A gate^T) * (A up^T), bfloat16.  Returns 0 when the
// fused kernel was launched, -1 when this problem is not taken (too few features to fill the GPU
// without a K split, or many tokens and a plan that splits K): the caller then runs the product
// and the activation apart.
FL_API int fl_gemm_tc_swiglu(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int I,
                             int K, int num_sms, int* status, cudaStream_t stream) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    // Up to 128 tokens: the one-tile kernel with as few features per CTA (16 to 64 in steps of 8) as
    // still leave every CTA a place on the SMs at once (two per SM); declined when even that gives too
    // few CTAs to keep the memory busy (a split of K does that better, with the activation apart).
    // Above: the CTA-pair kernel when the plan for the [2 I, K] product has no K split.
    int bn = 16, feat = 64;
    if (M <= 128) {
        while (bn < M) bn *= 2;
        feat = 16;
        while (feat < 64 && (I + feat - 1) / feat > 2 * num_sms) feat += 8;
        if ((I + feat - 1) / feat < (num_sms + 1) / 2) return -1;
    } else {
        int splits = 0;
        plan_one_tile(M, 2 * I, K, num_sms, &bn, &splits);      // (the pair kernel's narrower tiles have no gated form)
        if (splits != 1 || bn != 512) return -1;
    }
    CUtensorMap map_w, map_a;
    int rc = make_w_map(&map_w, W, 2L * I, K, ldw, feat);           // boxes of `feat` weight rows
    if (rc) return rc;
    const int wp = ldw == 0 ? 2 * I : 0;
    rc = make_map(&map_a, A, M, K, lda, bn > 256 ? tc_pair_tile_tokens(M, 256) / 2 : bn);
    if (rc) return rc;
    if (bn == 512)
        return launch_tc_pair<256, bf16, true>(map_w, map_a, C, ldc, M, I, K, num_sms, status, stream, I, 1, 0, nullptr, 0, nullptr, wp);
    const int kb = (K + TC_BK - 1) / TC_BK;
    switch (bn) {
        case 16: return launch_tc<16, 6, bf16, true>(map_w, map_a, C, ldc, nullptr, 0, M, I, K, 1, kb, status, stream, I, feat, wp);
        case 32: return launch_tc<32, 5, bf16, true>(map_w, map_a, C, ldc, nullptr, 0, M, I, K, 1, kb, status, stream, I, feat, wp);
        case 64: return launch_tc<64, 4, bf16, true>(map_w, map_a, C, ldc, nullptr, 0, M, I, K, 1, kb, status, stream, I, feat, wp);
        case 128: return launch_tc<128, 3, bf16, true>(map_w, map_a, C, ldc, nullptr, 0, M, I, K, 1, kb, status, stream, I, feat, wp);
    }
    return -1;
}

// The q|k|v product of an attention layer with its rotary encoding and cache write in the epilogue (see TcRope):
// W is [(n_heads + 2 n_kv_heads) * 128, K], q|k|v head-major; the rotated queries go to C[M, n_heads * 128]
// (row pitch ldc), rotated keys and the values into the cache slots of the tokens.  Returns 0 when launched and
// -1 when this problem is not taken (heads not of 128 rotated in full, 64 tokens or fewer, a plan that splits K,
// an output that is not 16-byte aligned): the caller then runs the product and the rotary kernel apart.
FL_API int fl_gemm_tc_qkv_rope(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int K,
                               int n_heads, int n_kv_heads, int head_dim, int rot_dim, const int* positions,
                               const int* slots, const float* cos_table, const float* sin_table, void* k_cache,
                               void* v_cache, long page_stride, int page_size, int num_sms, int* status,
                               cudaStream_t stream) {
    if (M <= 0) return 0;
    if (K <= 0 || n_heads <= 0 || n_kv_heads <= 0) return (int)cudaErrorInvalidValue;
    if (head_dim != 128 || rot_dim != 128 || M <= 64 || num_sms < 2 || k_cache == nullptr || v_cache == nullptr) return -1;
    if ((ldc % 8) || ((uintptr_t)C & 15) || (page_stride % 8) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return -1;
    const int N = (n_heads + 2 * n_kv_heads) * 128;
    // taken when the pair kernel over whole K costs no more than the cheapest product whose partial sums the
    // rotary kernel would add up, plus that kernel (about 3 us)
    const int bnt = M <= 128 ? 128 : 256;
    int bn = 0, splits = 0;
    fl_gemm_tc_plan_for(M, N, K, num_sms, 1, &bn, &splits);
    if (tc_cost(M, N, K, num_sms, bnt == 256 ? 512 : 640, 1, 1) > tc_cost(M, N, K, num_sms, bn, splits, 1) + 3.0) return -1;
    CUtensorMap map_w, map_a;
    int rc = make_w_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc) return rc;
    const int wp = ldw == 0 ? N : 0;
    rc = make_map(&map_a, A, M, K, lda, tc_pair_tile_tokens(M, bnt) / 2);
    if (rc) return rc;
    TcRope rope = {positions, slots, cos_table, sin_table, (bf16*)k_cache, (bf16*)v_cache, page_stride, page_size,
                   n_heads, n_kv_heads};
    switch (bnt) {
        case 64: return launch_tc_pair<64, bf16, false, true>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, 1, 0, nullptr, 0, &rope, wp);
        case 128: return launch_tc_pair<128, bf16, false, true>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, 1, 0, nullptr, 0, &rope, wp);
        case 256: return launch_tc_pair<256, bf16, false, true>(map_w, map_a, C, ldc, M, N, K, num_sms, status, stream, 0, 1, 0, nullptr, 0, &rope, wp);
    }
    return -1;
}

// ------------------------------------------- entry point that allocates nothing
// See gemm_tcgen05_static.h: the split-K workspace is this file-scope array, so
// a caller that cannot allocate can still use the split-K product.
#include <stdio.h>

#include "gemm_tcgen05_static.h"

#define FL_TC_MAX_DEVICES 64

static __device__ __align__(256) float tc_static_scratch[FL_TC_STATIC_SCRATCH_FLOATS];
// Device address of the array on each device; found at the first call there.
// `tc_static_scratch` itself is only a host-side handle in host code.
static float* tc_static_scratch_addr[FL_TC_MAX_DEVICES];

static void tc_say(char* text, int bytes, const char* fmt, long a, long b) {
    if (text != nullptr && bytes > 0) snprintf(text, (size_t)bytes, fmt, a, b);
}

FL_API int fl_gemm_tc_static_scratch(const void* A, long lda, const void* W, long ldw, void* C,
                                     int c_dtype, long ldc, int M, int N, int K, int bn, int splits,
                                     int num_sms, int* status, cudaStream_t stream, char* error_text,
                                     int error_text_bytes) {
    if (error_text != nullptr && error_text_bytes > 0) error_text[0] = '\0';
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= FL_TC_MAX_DEVICES) {
        tc_say(error_text, error_text_bytes, "device %ld is beyond the %ld devices this entry point tracks",
               (long)device, (long)FL_TC_MAX_DEVICES);
        return FL_TC_ERR_BAD_DEVICE;
    }
    if (tc_static_scratch_addr[device] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, tc_static_scratch);
        if (e != cudaSuccess) return (int)e;
        tc_static_scratch_addr[device] = p;
    }
    if (bn == 0) fl_gemm_tc_plan(M, N, K, num_sms, &bn, &splits);     // the rule of fl_gemm_tc: only bn == 0 plans
    if (splits < 1) return (int)cudaErrorInvalidValue;
    const long ld_partial = ((long)N + 3) / 4 * 4;
    const long needed = splits > 1 ? (long)splits * M * ld_partial : 0;
    if (needed > FL_TC_STATIC_SCRATCH_FLOATS) {
        tc_say(error_text, error_text_bytes,
               "this product needs %ld floats of split-K scratch; the built-in array holds %ld "
               "(use fewer splits, fewer tokens per call, or fl_gemm_tc with a workspace of your own)",
               needed, (long)FL_TC_STATIC_SCRATCH_FLOATS);
        return FL_TC_ERR_SCRATCH_TOO_SMALL;
    }
    return fl_gemm_tc(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, bn, splits, tc_static_scratch_addr[device],
                      FL_TC_STATIC_SCRATCH_FLOATS, num_sms, status, stream);
}
