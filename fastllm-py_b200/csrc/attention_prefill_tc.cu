// Paged causal attention for prompt portions on the Blackwell tensor cores:
// both products (Q K^T and P V) are tcgen05.mma with the accumulators in tensor
// memory; keys, values and queries arrive by TMA; the softmax runs in float on
// FT_PARTS threads per query row.
//
// A CTA takes 128 consecutive query rows of one request and one query head and
// walks the request's keys in blocks of 128 (starting at multiples of 128 of the
// absolute position, so a row's sequence of partial maxima does not depend on
// how the prompt was cut).  Per block:
//   producer warps  TMA: the block's pages of this head's keys (one warp) and values
//                   (another) into two-stage rings (one box of page_size x 64
//                   per page and 64 columns, each issued by a lane of its own;
//                   pages that do not exist are fetched from beyond the tensor,
//                   which fills zeros);
//   MMA warp        S = Q K^T into one of two S buffers in tensor memory (so the
//                   next block's scores are computed while this block's are
//                   being exponentiated), then O_blk = P V;
//   softmax warps   FT_PARTS threads share query row r: each reads its part of the row of S
//                   (tcgen05.ld), masks, exchanges the part's maximum with its
//                   partners, keeps the running maximum and sum in float, writes
//                   its part of P as bfloat16 into shared memory in the swizzled
//                   K-major layout the second MMA reads, and adds its columns
//                   of O_blk into its part of the output row, which it holds in
//                   registers (rescaled when the maximum moves).
// Every wait on an mbarrier is bounded; a give-up sets an error word and all
// roles leave.
//
// fastllm-py's counterpart is `_sdpa` (fastllm_py/model.py:341-353).  The
// mma.sync kernel in attention_prefill.cu computes the same thing and serves the
// head sizes and page sizes this one does not take (HEAD_DIM 64 or 128; page
// sizes that are multiples of 8 and divide 128).
#include <cuda.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the tcgen05 prefill kernel takes head sizes 64 and 128");

#define FT_BM 128                          // query rows per CTA
#define FT_BN 128                          // keys per block
#ifndef FT_STAGES
#define FT_STAGES 3                        // key and value ring depth (each)
#endif
#ifndef FT_PARTS
#define FT_PARTS 2                         // softmax threads per query row
#endif
#define FT_KP (FT_BN / FT_PARTS)           // keys of a block per softmax thread
#define FT_OD (HEAD_DIM / FT_PARTS)        // output columns per softmax thread
static_assert(FT_OD % 32 == 0 && FT_KP % 32 == 0, "a softmax thread owns multiples of 32 keys and of 32 columns");
#define FT_SOFTMAX_THREADS (128 * FT_PARTS)
#define FT_SOFTMAX_WARPS (FT_SOFTMAX_THREADS / 32)
#define FT_PRODUCER_WARP FT_SOFTMAX_WARPS                      // queries and keys
#define FT_MMA_WARP (FT_SOFTMAX_WARPS + 1)
#define FT_VPRODUCER_WARP (FT_SOFTMAX_WARPS + 2)              // values
#define FT_THREADS ((FT_SOFTMAX_WARPS + 3) * 32)
#define FT_ATOMS (HEAD_DIM / 64)           // 64-column swizzle atoms per row
#define FT_ATOM_BYTES (128 * 128)          // 128 rows x 128 bytes
#define FT_WAIT_LIMIT_NS 2000000000ull

enum { FT_ERR_WAIT = 301, FT_ERR_SMEM = 302 };

// ------------------------------------------------------------------ PTX wraps
__device__ __forceinline__ uint32_t ft_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ft_bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ft_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ft_bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ft_smem(bar)) : "memory");
}
__device__ __forceinline__ void ft_bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ft_smem(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint64_t ft_now() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool ft_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    uint32_t ok = 0, spins = 0;
    uint64_t t0 = 0;
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(ft_smem(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((++spins & 127u) == 0) {
            if (*abort_flag) return false;
            if (t0 == 0) t0 = ft_now();
            else if (ft_now() - t0 > FT_WAIT_LIMIT_NS) return false;
        }
    }
}
// A warp waits through its first lane and arrives through it (after __syncwarp, which orders
// the other lanes' writes before the arrival): a barrier then sees 8 arrivals per phase from the
// softmax warps instead of 256, and one thread polls instead of 32.
__device__ __forceinline__ bool ft_warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = ft_wait(bar, parity, abort_flag) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void ft_warp_arrive(uint64_t* bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) ft_bar_arrive(bar);
}
__device__ __forceinline__ void ft_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(ft_smem(dst)),
        "l"((uint64_t)map), "r"(ft_smem(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void ft_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ft_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ft_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void ft_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ft_smem(bar))
                 : "memory");
}
__device__ __forceinline__ void ft_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void ft_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void ft_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void ft_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows in the lanes, 16 bfloat16 of K as 8 columns) comes
// from tensor memory
__device__ __forceinline__ void ft_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// K-major operand, rows of 128 bytes in the 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t ft_desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (the contiguous axis is N): 64-element blocks of N are FT_ATOM_BYTES apart
// (leading offset), groups of 8 K rows 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t ft_desc_mnmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(FT_ATOM_BYTES >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// float accumulator, bfloat16 operands; b_mn: B is MN-major
__host__ __device__ constexpr uint32_t ft_idesc(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
// 2^x by the special-function unit (relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float ft_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ft_weight(float a, float b) { return (a == -CUDART_INF_F) ? 0.0f : exp2f(a - b); }

struct FtSmem {
    static constexpr int Q_BYTES = FT_ATOMS * FT_ATOM_BYTES;
    static constexpr int KV_BYTES = FT_ATOMS * FT_ATOM_BYTES;          // one of K or V, one stage
    static constexpr int TILES = Q_BYTES + 2 * FT_STAGES * KV_BYTES;
    static constexpr int BAR_SLOTS = 24 + 4 * FT_STAGES;               // 8-byte slots: barriers and the like
    static constexpr int BARS = BAR_SLOTS * 8 + 2 * FT_PARTS * 128 * 4; // ... then the parts' maxima (two rounds)
    // The tiles want a 1024-byte boundary.  Where they fill the SM's shared memory to within a KB
    // there is no room to round up to one: the kernel then counts on the dynamic shared memory
    // starting on such a boundary (it has no static shared memory) and reports FT_ERR_SMEM instead
    // of running if it does not.
    static constexpr int SLACK = (TILES + BARS + 1024 <= 232448) ? 1024 : 0;
    static constexpr int TOTAL = TILES + BARS + SLACK;
};

__global__ void __launch_bounds__(FT_THREADS, 1) attention_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
    bf16* __restrict__ out, long out_ld, int page_size, int kv_rows_total, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ req_start, const int* __restrict__ req_ctx,
    const int* __restrict__ req_qlen, int n_requests, int include_single, int n_heads, int n_kv_heads,
    int window, float scale_log2e, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char ft_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)ft_raw + 1023) & ~(uintptr_t)1023);
    if (base + FtSmem::TILES + FtSmem::BARS > ft_raw + FtSmem::TOTAL) {       // uniform over the CTA
        if (threadIdx.x == 0) atomicCAS(status, 0, FT_ERR_SMEM);
        return;
    }
    unsigned char* q_s = base;
    unsigned char* k_s = q_s + FtSmem::Q_BYTES;                        // [stage][atom][128 rows][128 B]
    unsigned char* v_s = k_s + FT_STAGES * FtSmem::KV_BYTES;
    uint64_t* bars = (uint64_t*)(base + FtSmem::TILES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 24;                                      // [FT_STAGES]
    uint64_t* k_empty = k_full + FT_STAGES;
    uint64_t* s_full = bars + 5;                                       // [2]
    uint64_t* p_full = bars + 9;                                       // [2]
    uint64_t* o_done = bars + 11;
    uint32_t* tmem_slot = (uint32_t*)(bars + 13);
    uint64_t* x_bar = bars + 14;                                       // the softmax threads' exchange point
    uint64_t* v_full = k_empty + FT_STAGES;
    uint64_t* v_empty = v_full + FT_STAGES;
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    volatile int* never = (volatile int*)(bars + 15);                  // stays 0: for waits that must not be cut short

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp == FT_PRODUCER_WARP || warp == FT_VPRODUCER_WARP;
    if (producer && lane == 0) {
        // the copies' descriptors are wanted first thing: ask for them while the tile is being worked out
        if (warp == FT_PRODUCER_WARP) asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_kv) : "memory");
    }
    // which request and which 128-row tile: blockIdx.y counts tiles, a request's last (longest) tile first
    int req = -1, tile = 0;
    {
        int acc = 0;
        for (int r = 0; r < n_requests; ++r) {
            const int ql = req_qlen[r];
            const int nt = (ql > 1 || include_single) ? (ql + FT_BM - 1) / FT_BM : 0;
            if ((int)blockIdx.y < acc + nt) { req = r; tile = nt - 1 - ((int)blockIdx.y - acc); break; }
            acc += nt;
        }
    }
    if (req < 0) return;
    const int h = blockIdx.x;
    const int kvh = h / (n_heads / n_kv_heads);
    const int q_len = req_qlen[req], ctx = req_ctx[req], row0 = tile * FT_BM;
    const int tok0 = req_start[req] + row0;
    const int rows_here = min(FT_BM, q_len - row0);
    const int pos_first = ctx + row0, pos_last = ctx + row0 + rows_here - 1;
    const int lo_tile = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int kb_begin = lo_tile / FT_BN, kb_end = pos_last / FT_BN + 1;
    const int n_blocks = kb_end - kb_begin;

    // ---- the producers' side of a block: one box of a page and 64 columns per lane.  A block of 128 keys is
    // pages x atoms boxes of a few KB; one lane issues one box (looking up its page itself), so a block's
    // copies leave together.
    const int is_v = warp == FT_VPRODUCER_WARP ? 1 : 0;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    auto issue_block = [&](int i) {
        unsigned char* ring = is_v ? v_s : k_s;
        const int* bt = block_table + (long)req * bt_stride;
        const int n_ops = (FT_BN / page_size) * FT_ATOMS;
        const int s = i % FT_STAGES;
        if (lane == 0) ft_bar_expect(&full[s], FtSmem::KV_BYTES);
        __syncwarp();
        const int key0 = (kb_begin + i) * FT_BN;
        for (int op = lane; op < n_ops; op += 32) {
            const int p = op / FT_ATOMS, a = op % FT_ATOMS;
            const int first_key = key0 + p * page_size;
            const int last_key = first_key + page_size - 1;
            // a page wholly outside what this tile may see is fetched from beyond the tensor: zeros
            int row = kv_rows_total;
            if (first_key <= pos_last && last_key >= lo_tile) {
                const long pg = bt[first_key / page_size];
                row = (int)(((pg * 2 + is_v) * n_kv_heads + kvh) * page_size);
            }
            const int off = s * FtSmem::KV_BYTES + a * FT_ATOM_BYTES + p * page_size * 128;
            ft_tma_2d(ring + off, &map_kv, &full[s], a * 64, row);
        }
    };
    // The producer warps set up their own barriers and send for the queries and the first block (the rings are
    // empty: nothing to wait for) before the CTA meets for the rest of its set-up, which the copies' way through
    // memory then hides: tensor memory, the other barriers, a look at the error word.  A tile with many blocks
    // sends for a whole ring at once; for a short one that only put the queries, which are wanted first, behind
    // three blocks of keys and values (measured: 2048 tokens 76 us against 70, 8192 tokens 693 against 744).
    const int early = n_blocks > 32 ? FT_STAGES : 1;
    int issued = 0;
    if (producer) {
        if (lane == 0) {
            if (!is_v) ft_bar_init(q_full, 1);
            for (int s = 0; s < FT_STAGES; ++s) {
                ft_bar_init(&full[s], 1);
                ft_bar_init(&empty[s], 1);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (!is_v) {
                ft_bar_expect(q_full, FtSmem::Q_BYTES);
                for (int a = 0; a < FT_ATOMS; ++a)
                    ft_tma_2d(q_s + a * FT_ATOM_BYTES, &map_q, q_full, h * HEAD_DIM + a * 64, tok0);
            }
        }
        __syncwarp();
        for (; issued < n_blocks && issued < early; ++issued) issue_block(issued);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            ft_bar_init(&s_full[s], 1);
            ft_bar_init(&p_full[s], FT_SOFTMAX_WARPS);
        }
        ft_bar_init(o_done, 1);
        ft_bar_init(x_bar, FT_SOFTMAX_WARPS);
        *abort_flag = (*(volatile int*)status != 0) ? 1 : 0;
        *never = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == FT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ft_smem(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ft_fence_before();
    __syncthreads();
    ft_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem;                                      // two S buffers: columns 0 and 128
    const uint32_t tmem_o = tmem + 256;                                // O: HEAD_DIM columns, accumulated over the blocks

#define FT_GIVE_UP()                                                             \
    {                                                                            \
        if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, FT_ERR_WAIT); } \
        break;                                                                   \
    }

    if (producer) {
        // ---- producers: one warp for the queries and the keys, one for the values, each with a ring of its
        // own.  A key stage is free again as soon as S of its block is computed, which is a whole block
        // earlier than P V; with keys and values in one ring the next keys could only be asked for after
        // P V, and their way through TMA showed.
        int i = issued;
        for (; i < n_blocks && !*abort_flag; ++i) {
            if (!ft_warp_wait(&empty[i % FT_STAGES], ((uint32_t)(i / FT_STAGES) & 1u) ^ 1u, abort_flag)) FT_GIVE_UP();
            issue_block(i);
        }
        if (*abort_flag) {
            // leaving early: the copies still on their way must land before the shared memory goes to
            // another CTA (the wait is bounded like every other)
            for (int k = max(0, i - FT_STAGES); k < i; ++k)
                ft_warp_wait(&full[k % FT_STAGES], (uint32_t)(k / FT_STAGES) & 1u, never);
            if (!is_v && lane == 0) ft_wait(q_full, 0, never);
        }
    } else if (warp == FT_MMA_WARP) {
        if (lane == 0 && !*abort_flag) {
            // ---- MMA issuer.  The tensor core runs what this thread issues in order, so S(i + 2),
            // which goes where S(i) and then P(i) were, follows P V of block i without a barrier.
            constexpr uint32_t idesc_s = ft_idesc(FT_BM, FT_BN, 0);
            constexpr uint32_t idesc_o = ft_idesc(FT_BM, HEAD_DIM, 1);
            auto issue_s = [&](int i) -> bool {                        // S(i) = Q K(i)^T into S buffer i & 1
                const int s = i & 1, ks = i % FT_STAGES;
                if (!ft_wait(&k_full[ks], (uint32_t)(i / FT_STAGES) & 1u, abort_flag)) return false;
                ft_fence_after();
                const uint32_t qa = ft_smem(q_s), ka = ft_smem(k_s + ks * FtSmem::KV_BYTES);
#pragma unroll
                for (int k = 0; k < HEAD_DIM / 16; ++k) {
                    const uint32_t off = (uint32_t)((k >> 2) * FT_ATOM_BYTES + (k & 3) * 32);
                    ft_mma(tmem_s + (uint32_t)(s * FT_BN), ft_desc_kmajor(qa + off), ft_desc_kmajor(ka + off),
                           idesc_s, k > 0 ? 1u : 0u);
                }
                ft_commit(&k_empty[ks]);            // the key stage is free once these MMAs have read it
                ft_commit(&s_full[s]);
                return true;
            };
            bool ok = ft_wait(q_full, 0, abort_flag);
            if (ok) ok = issue_s(0);
            for (int i = 0; i < n_blocks && ok; ++i) {
                // S(i + 1) overwrites buffer (i + 1) & 1, which held S(i - 1) and P(i - 1): the wait on
                // p_full of block i - 1 (a round ago) says the softmax has read that S, and P V of block
                // i - 1 was issued before this
                if (i + 1 < n_blocks && !issue_s(i + 1)) { ok = false; break; }
                const int b = i & 1, vs = i % FT_STAGES;
                if (!ft_wait(&v_full[vs], (uint32_t)(i / FT_STAGES) & 1u, abort_flag)) { ok = false; break; }
                if (!ft_wait(&p_full[b], (uint32_t)(i >> 1) & 1u, abort_flag)) { ok = false; break; }
                ft_fence_after();
                // O (+)= P(i) V(i): A = P from tensor memory (rows in the lanes, 16 keys = 8 columns of
                // bfloat16 pairs, at the start of S buffer b); B = V: MN-major, 16 keys = two 8-row groups
                const uint32_t pa = tmem_s + (uint32_t)(b * FT_BN), va = ft_smem(v_s + vs * FtSmem::KV_BYTES);
#pragma unroll
                for (int k = 0; k < FT_BN / 16; ++k)
                    ft_mma_ts(tmem_o, pa + (uint32_t)(k * 8), ft_desc_mnmajor(va + (uint32_t)(k * 16 * 128)), idesc_o,
                              (i > 0 || k > 0) ? 1u : 0u);
                ft_commit(&v_empty[vs]);
                ft_commit(o_done);                  // phase i: O holds the blocks up to i
            }
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, FT_ERR_WAIT); }
        }
    } else {
        // ---- softmax: FT_PARTS threads (r, r + 128, ...) share query row r; `part` says which
        // FT_KP keys of a block and which FT_OD output columns a thread owns.  P goes back into
        // tensor memory, over the first half of the S it was made from, as the A operand of P V,
        // and O stays in tensor memory, where P V accumulates; it is rescaled (read, multiplied,
        // written back by these threads) only when a row's maximum has grown by more than 2^8
        // since the scale in use was set: until then the exponentials simply use the older maximum
        // (they stay below 2^8, well inside bfloat16 and float), and no thread waits for P V.
        const int r = threadIdx.x & 127;
        const int part = threadIdx.x >> 7;
        const int pos_r = ctx + row0 + r;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        // [round parity][part][row]: a round's values stay untouched while the next round's are written
        float* part_max_all = reinterpret_cast<float*>(bars + FtSmem::BAR_SLOTS);
        float m_run = -CUDART_INF_F, l_run = 0.0f;           // m_run: the maximum the scale in use is based on
        bool ok = !*abort_flag;
        for (int i = 0; i < n_blocks && ok; ++i) {
            const int sb = i & 1;
            if (!ft_warp_wait(&s_full[sb], (uint32_t)(i >> 1) & 1u, abort_flag)) FT_GIVE_UP();
            ft_fence_after();
            const int key0 = (kb_begin + i) * FT_BN + part * FT_KP;      // first key of this thread's part
            const uint32_t s_addr = tmem_s + (uint32_t)(sb * FT_BN + part * FT_KP) + lane_base;
            const bool all_seen = (key0 + FT_KP - 1 <= pos_r) && (window <= 0 || key0 > pos_r - window);
            uint32_t v[FT_KP];
#pragma unroll
            for (int c = 0; c < FT_KP; c += 32) ft_ld32(s_addr + (uint32_t)c, v + c);
            ft_ld_wait();
            if (!all_seen) {
#pragma unroll
                for (int j = 0; j < FT_KP; ++j) {
                    const int key = key0 + j;
                    if (!(key <= pos_r && (window <= 0 || key > pos_r - window))) v[j] = 0xff800000u;   // -inf
                }
            }
            float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int j = 0; j < FT_KP; j += 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], __uint_as_float(v[j + e]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // exchange the parts' maxima (one barrier among the softmax warps per block); past it
            // every softmax thread has its S in registers, so the S buffer may take P
            float* part_max = part_max_all + (i & 1) * (FT_PARTS * 128);
            part_max[part * 128 + r] = mx;
            ft_warp_arrive(x_bar);                                        // (an mbarrier: its wait can give up)
            if (!ft_warp_wait(x_bar, (uint32_t)i & 1u, abort_flag)) FT_GIVE_UP();
            float mx_row = part_max[r];
#pragma unroll
            for (int q = 1; q < FT_PARTS; ++q) mx_row = fmaxf(mx_row, part_max[q * 128 + r]);
            const float m_new = fmaxf(m_run, mx_row * scale_log2e);
            // the row's threads decide alike: they see the same maxima
            const bool rescale = m_new > m_run + 8.0f || (m_run == -CUDART_INF_F && m_new != -CUDART_INF_F);
            const bool any_rescale = __any_sync(0xffffffffu, rescale);
            float corr = 1.0f;
            if (rescale) {
                corr = ft_weight(m_run, m_new);
                l_run *= corr;
                m_run = m_new;
            }
            if (any_rescale && i > 0) {
                // O holds blocks 0 .. i - 1 once P V of block i - 1 is complete.  The whole warp reads,
                // scales and writes its rows back (rows that keep their scale by 1): the loads and
                // stores of tensor memory are warp-wide instructions.
                if (!ft_warp_wait(o_done, (uint32_t)(i - 1) & 1u, abort_flag)) FT_GIVE_UP();
                ft_fence_after();
#pragma unroll
                for (int c = 0; c < FT_OD; c += 32) {
                    uint32_t w[32];
                    const uint32_t o_addr = tmem_o + lane_base + (uint32_t)(part * FT_OD + c);
                    ft_ld32(o_addr, w);
                    ft_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(w[j]) * corr);
                    ft_st32(o_addr, w);
                }
            }
            const float neg_m = (m_run == -CUDART_INF_F) ? 0.0f : -m_run;      // an empty row: every p below is 0
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t packed[FT_KP / 2];
#pragma unroll
            for (int c = 0; c < FT_KP / 2; ++c) {
                const float p0 = ft_ex2(fmaf(__uint_as_float(v[2 * c]), scale_log2e, neg_m));
                const float p1 = ft_ex2(fmaf(__uint_as_float(v[2 * c + 1]), scale_log2e, neg_m));
                l4[c & 3] += p0 + p1;
                const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                packed[c] = *reinterpret_cast<const uint32_t*>(&b);
            }
            l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            // P(i): this thread's FT_KP keys as FT_KP / 2 columns of bfloat16 pairs
#pragma unroll
            for (int c = 0; c < FT_KP / 2; c += 32)
                ft_st32(tmem_s + (uint32_t)(sb * FT_BN + part * (FT_KP / 2) + c) + lane_base, packed + c);
            ft_st_wait();
            ft_fence_before();
            ft_warp_arrive(&p_full[sb]);
        }
        // the whole of O, then the row's sum: the parts' sums (all relative to the same maximum)
        if (ok && n_blocks > 0) {
            ok = ft_warp_wait(o_done, (uint32_t)(n_blocks - 1) & 1u, abort_flag);
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, FT_ERR_WAIT); }
            ft_fence_after();
        }
        float* part_sum = part_max_all + (n_blocks & 1) * (FT_PARTS * 128);
        part_sum[part * 128 + r] = l_run;
        ft_warp_arrive(x_bar);
        const bool met = ft_warp_wait(x_bar, (uint32_t)n_blocks & 1u, abort_flag);
        float l_row = part_sum[r];
#pragma unroll
        for (int q = 1; q < FT_PARTS; ++q) l_row += part_sum[q * 128 + r];
        if (met && ok && !*abort_flag && n_blocks > 0) {
            const float inv = 1.0f / l_row;
            bf16* dst = out + (long)(tok0 + r) * out_ld + (long)h * HEAD_DIM + part * FT_OD;
#pragma unroll
            for (int c = 0; c < FT_OD; c += 32) {
                uint32_t w[32];
                ft_ld32(tmem_o + lane_base + (uint32_t)(part * FT_OD + c), w);      // all lanes of the warp take part
                ft_ld_wait();
                if (r < rows_here) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 o4;
                        __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            wp[e] = __floats2bfloat162_rn(__uint_as_float(w[d + 2 * e]) * inv,
                                                          __uint_as_float(w[d + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + d) = o4;
                    }
                }
            }
        }
    }
#undef FT_GIVE_UP
    ft_fence_before();
    __syncthreads();
    if (warp == FT_MMA_WARP) {
        ft_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ----------------------------------------------------------------- host side
typedef CUresult (*FtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FtEncodeFn ft_encode_fn() {
    static FtEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (FtEncodeFn)p;
    }
    return fn;
}
static int ft_make_map(CUtensorMap* map, const void* base, long rows, long cols, long ld, int box_rows) {
    FtEncodeFn fn = ft_encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    if (((uintptr_t)base & 15) || ((ld * 2) & 15)) return (int)cudaErrorMisalignedAddress;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

FL_API int fl_attention_prefill_tc_head_dim() { return HEAD_DIM; }
FL_API int fl_attention_prefill_tc_takes(int page_size) {
    return page_size >= 8 && page_size <= FT_BN && page_size % 8 == 0 && FT_BN % page_size == 0;
}

// The arguments of fl_attention_prefill (attention_prefill.cu) with the cache given
// as one tensor [n_pages, 2, n_kv_heads, page_size, HEAD_DIM] and a status word.
FL_API int fl_attention_prefill_tc(const void* q, long q_ld, void* out, long out_ld, const void* cache,
                                   long n_pages, int page_size, const int* block_table, int bt_stride,
                                   const int* req_start, const int* req_ctx, const int* req_qlen,
                                   int n_requests, int n_tokens, int include_single, int n_heads,
                                   int n_kv_heads, int window, float scale, int* status, cudaStream_t stream) {
    if (n_requests <= 0 || n_tokens <= 0) return 0;
    if (!fl_attention_prefill_tc_takes(page_size) || n_heads > 65535 || n_heads % n_kv_heads)
        return (int)cudaErrorInvalidValue;
    if ((q_ld % 8) || (out_ld % 8)) return (int)cudaErrorMisalignedAddress;
    const long kv_rows = n_pages * 2 * n_kv_heads * page_size;
    if (kv_rows >= (1l << 31)) return (int)cudaErrorInvalidValue;
    CUtensorMap map_q, map_kv;
    int rc = ft_make_map(&map_q, q, n_tokens, (long)n_heads * HEAD_DIM, q_ld, FT_BM);
    if (rc) return rc;
    rc = ft_make_map(&map_kv, cache, kv_rows, HEAD_DIM, HEAD_DIM, page_size);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             FtSmem::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int max_tiles = n_tokens / FT_BM + n_requests;
    if (max_tiles > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(n_heads, max_tiles);                 // heads fastest: every head's late (long) tiles start first
    // plain stream order (no programmatic overlap): this kernel takes all of an SM's tensor memory
    attention_prefill_tc_kernel<<<grid, FT_THREADS, FtSmem::TOTAL, stream>>>(
        map_q, map_kv, (bf16*)out, out_ld, page_size, (int)kv_rows, block_table, bt_stride, req_start, req_ctx,
        req_qlen, n_requests, include_single, n_heads, n_kv_heads, window, scale * 1.4426950408889634f, status);
    return fl_launch_status();
}
