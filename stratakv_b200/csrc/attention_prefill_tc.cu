// Prefill attention on the 5th-generation tensor cores (bfloat16, head size 64 or 128): causal
// grouped-query flash attention over the paged cache with both matrix products in tcgen05.mma.
//
// It does the arithmetic of attention_prefill.cu (src/layers/attention.cpp:261-338 in the
// reference, which has no prefill kernel at all) with another division of labour.  A block takes
// 128 queries of one head; keys and values come in tiles of 64 positions:
//   warp 0   keys and scores: TMA loads of the Q tile (once) and of K tiles into a ring of four stages (a tile
//            is gathered from the cache blocks the sequence's block table names, whose entries the warp holds 32
//            at a time in registers), and S = Q.K^T (128 x 64 x head_dim) into one of two score buffers in
//            tensor memory, a tile ahead of the softmax;
//   warp 1   values and output: TMA loads of V tiles into a ring of three stages, and O += P.V
//            (128 x head_dim x 64) into the output accumulator, also in tensor memory; V is used as it lies
//            in the cache (positions x head_dim), as an MN-major operand.
//            Both warps walk their loops whole, and one elected lane issues.  A single issuing thread for
//            both products measured as the limit of the kernel: its four waits and sixteen small tcgen05
//            instructions a tile took 1,800 cycles, more than the softmax of the tile;
//   warps 2-5  one thread per query row: read the scores with tcgen05.ld, mask, 2^x on the
//            special-function unit (scores carry log2 e), row sums, probabilities as bfloat16 into
//            one of two swizzled shared-memory tiles (the A operand of P.V).  The maximum the
//            exponentials are taken against is raised only when a tile exceeds it by 2^8; only then
//            is the accumulated output rescaled (tcgen05.ld / st), so most tiles never touch it.
//            At the end the output is read once, divided by the row sum and stored.
// The softmax is the long pole, so a block uses only half of the SM's tensor memory and shared
// memory and (for head size 64) two blocks share an SM.  Every mbarrier
// wait is bounded; on time-out bit 2 (value 4) of the flag word is raised and the block drains.
#include "common.cuh"

#if SKV_DTYPE == SKV_BF16 && (SKV_HEAD_DIM == 64 || SKV_HEAD_DIM == 128)

#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <utility>
#include <vector>

namespace skv {

constexpr int AHD = SKV_HEAD_DIM;
constexpr int ACH = AHD / 64;                       // 64-wide (128-byte) chunks of a head
constexpr int ABM = 128, ABN = 64;                  // queries and keys per tile
constexpr int ATHREADS = 192;
constexpr uint32_t AWAIT = 1u << 20;
constexpr uint32_t TILE_BYTES = 128 * 128;          // one 128-row x 128-byte swizzled tile
constexpr uint32_t KV_TILE_BYTES = ABN * 128;       // one 64-row tile of keys or values

__device__ __forceinline__ uint32_t a_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void a_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void a_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void a_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool a_wait(uint32_t bar, uint32_t parity, int* flag) {
    for (uint32_t tries = 0; tries < AWAIT; ++tries) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    if (flag) atomicOr(flag, 4);
    return false;
}
// One lane of a converged warp (the compiler can then keep what the issuing lane computes in uniform registers)
__device__ __forceinline__ bool a_elect() {
    uint32_t chosen;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    return chosen != 0;
}
__device__ __forceinline__ void a_tma(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// 128-byte-swizzled tile with 128-byte rows; 1024 bytes between groups of 8 rows (see gemm_tcgen05.cu)
__device__ __forceinline__ uint64_t a_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, float accumulator, bfloat16 operands; b_mn = 1: B is MN-major (rows are the K index)
__device__ __forceinline__ constexpr uint32_t a_idesc(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void a_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void a_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void a_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ float a_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float a_max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}

__device__ __forceinline__ void a_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

// Keys come through a ring of four tiles and values through one of three, both asked for two tiles ahead (a stage of
// keys is known to be free when the softmax has taken the scores of its tile, a stage of values when the product after
// it has been seen complete); scores and probabilities have two buffers each.
constexpr int K_STAGES = 4, V_STAGES = 3;
// barriers: Q; K full and V full for each stage of the rings; S full/empty and P full/empty for each buffer
enum { B_Q = 0, B_KF = 1, B_VF = B_KF + K_STAGES, B_SF = B_VF + V_STAGES, B_SE = B_SF + 2, B_PF = B_SE + 2, B_PE = B_PF + 2,
       B_COUNT = B_PE + 2 };

// The running maximum a row's exponentials are taken against is only raised when a tile's maximum
// exceeds it by more than this many powers of two; until then the accumulated output (in tensor
// memory) needs no rescaling and probabilities stay below 2^RESCALE_MARGIN.
constexpr float RESCALE_MARGIN = 8.0f;

__global__ void __launch_bounds__(ATHREADS, AHD <= 64 ? 2 : 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_after,
                            __nv_bfloat16* __restrict__ out, int num_heads, int num_kv_heads, int block_size,
                            int rows_per_load, float scale, int window, int tiles_per_seq, int* __restrict__ flag) {
    extern __shared__ uint8_t a_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)a_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = base;                                        // ACH tiles of 128 rows
    uint8_t* k_ring = q_tile + ACH * TILE_BYTES;                   // K_STAGES stages x ACH tiles of 64 rows
    uint8_t* v_ring = k_ring + K_STAGES * ACH * KV_TILE_BYTES;     // V_STAGES stages x ACH tiles of 64 rows
    uint8_t* p_ring = v_ring + V_STAGES * ACH * KV_TILE_BYTES;            // 2 tiles of 128 rows (64 keys = 128 bytes a row)
    uint64_t* bars = (uint64_t*)(p_ring + 2 * TILE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + B_COUNT);
    const uint32_t bar0 = a_smem(bars);
    auto bar = [&](int which, int index = 0) { return bar0 + 8u * (uint32_t)(which + index); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Heads run fastest (the heads of a KV head work on the same keys at the same time), and the query tiles
    // are handed out last first: under a causal mask the last tile of a prompt has the most keys, and the
    // blocks that start when the first ones have left should be the short ones.
    const int order = (int)(gridDim.y - 1 - blockIdx.y);
    const int seq = order / tiles_per_seq, tile = order - seq * tiles_per_seq;
    const int head = blockIdx.x;
    const int kv_head = head / (num_heads / num_kv_heads);
    pdl_launch_dependents();
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    if (tile * ABM >= q_len) return;                               // the whole block leaves together
    const int ctx = ctx_after[seq], ctx_before = ctx - q_len;
    const int last_query = min(q_len, tile * ABM + ABM) - 1;
    const int kv_end = ctx_before + last_query + 1;
    const int kv_lo = window > 0 ? max(0, ctx_before + tile * ABM - window + 1) : 0;
    const int first_tile = kv_lo / ABN, n_tiles = (kv_end + ABN - 1) / ABN - first_tile;

    if (threadIdx.x == 0) {
        a_init(bar(B_Q), 1);
        for (int i = 0; i < K_STAGES; ++i) a_init(bar(B_KF, i), 1);
        for (int i = 0; i < V_STAGES; ++i) a_init(bar(B_VF, i), 1);
        for (int i = 0; i < 2; ++i) {
            a_init(bar(B_SF, i), 1); a_init(bar(B_SE, i), 4); a_init(bar(B_PF, i), 4); a_init(bar(B_PE, i), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(a_smem(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;             // S: 2 x 64 columns; O: AHD columns
    pdl_wait();                                                    // q and the cache rows come from the kernels before

    // Cache rows of a tile of 64 keys, for the copies of either warp below: the block table's entries come 32 at a time
    // into one register per lane (a look-up per tile by the issuing lane alone would put the latency of a read from
    // global memory into every round of its loop).
    const int* table = block_table + (size_t)seq * table_width;
    int cached_from = -1, cached_entry = 0;
    auto cache_row = [&](int key) {                                    // called by the whole warp
        const int entry = key / block_size;
        if (cached_from < 0 || entry < cached_from || entry >= cached_from + 32) {
            cached_from = entry;
            cached_entry = table[min(entry + lane, table_width - 1)];
        }
        const int block = __shfl_sync(0xffffffffu, cached_entry, entry - cached_from);
        return (block * num_kv_heads + kv_head) * block_size + (key % block_size);
    };
    auto load_tile = [&](int which, int t) {                           // 0: keys, 1: values; tile t of this block
        const int st = which ? t % V_STAGES : t % K_STAGES;
        const uint32_t full = bar(which ? B_VF : B_KF, st);
        uint8_t* dst = (which ? v_ring : k_ring) + (size_t)st * ACH * KV_TILE_BYTES;
        const int key0 = (first_tile + t) * ABN;
        const bool issuer = a_elect();
        if (issuer) a_expect(full, ACH * KV_TILE_BYTES);
        for (int r = 0; r < ABN; r += rows_per_load) {
            const int row = cache_row(key0 + r);
            if (issuer) {
                for (int c = 0; c < ACH; ++c)
                    a_tma(a_smem(dst + c * KV_TILE_BYTES + r * 128), which ? &map_v : &map_k, 64 * c, row, full);
            }
        }
        __syncwarp();
    };
    if (warp == 0) {
        // ---- keys and scores: the whole warp walks the loop, one elected lane issues -----------------------
        // For tile i: wait until softmax i - 2 has taken its scores out of the buffer (which also says that the
        // product of tile i - 2 is complete and its keys' stage free), and for the keys of tile i; issue
        // S[i & 1] = Q . K_i^T; then ask for the keys of tile i + 2, into the stage of tile i - 2.
        if (a_elect()) {
            a_expect(bar(B_Q), ACH * TILE_BYTES);
            for (int c = 0; c < ACH; ++c)
                a_tma(a_smem(q_tile + c * TILE_BYTES), &map_q, head * AHD + 64 * c, q_begin + tile * ABM, bar(B_Q));
        }
        __syncwarp();
        for (int t = 0; t < 2 && t < n_tiles; ++t) load_tile(0, t);
        constexpr uint32_t idesc_s = a_idesc(ABM, ABN, 0);
        bool ok = a_wait(bar(B_Q), 0, flag);
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int s = i & 1, ks = i % K_STAGES;
            if (i >= 2) ok = a_wait(bar(B_SE, s), ((i >> 1) - 1) & 1, flag);
            if (ok) ok = a_wait(bar(B_KF, ks), (i / K_STAGES) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (a_elect()) {
#pragma unroll
                for (int c = 0; c < ACH; ++c) {
                    const uint64_t qd = a_desc(a_smem(q_tile + c * TILE_BYTES));
                    const uint64_t kd = a_desc(a_smem(k_ring + (size_t)(ks * ACH + c) * KV_TILE_BYTES));
#pragma unroll
                    for (int k = 0; k < 4; ++k) a_mma(tmem_s + 64u * s, qd + 2 * k, kd + 2 * k, idesc_s, (c | k) ? 1u : 0u);
                }
                a_commit(bar(B_SF, s));
            }
            __syncwarp();
            if (i + 2 < n_tiles) load_tile(0, i + 2);
        }
        if (!ok) {
            // a wait gave up: let the copies in flight land (microseconds) before the block may leave
            for (int t = 0; t < 64; ++t) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ---- values and output products: O += P_j . V_j once the probabilities and the values are in shared
        // memory; then the values of tile j + 2 are asked for, into the stage of tile j - 1, whose product (issued
        // a round ago) has to be complete.
        constexpr uint32_t idesc_o = a_idesc(ABM, 64, 1);
        for (int t = 0; t < 2 && t < n_tiles; ++t) load_tile(1, t);
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j & 1, vs = j % V_STAGES;
            ok = a_wait(bar(B_VF, vs), (j / V_STAGES) & 1, flag) && a_wait(bar(B_PF, s), (j >> 1) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (a_elect()) {
#pragma unroll
                for (int kk = 0; kk < ABN / 16; ++kk) {               // 16 keys per instruction
                    const uint64_t pd = a_desc(a_smem(p_ring + s * TILE_BYTES)) + 2 * kk;
#pragma unroll
                    for (int c = 0; c < ACH; ++c) {
                        // V tile rows are keys: 16 keys further is 16 x 128 bytes = 128 descriptor units
                        const uint64_t vd = a_desc(a_smem(v_ring + (size_t)(vs * ACH + c) * KV_TILE_BYTES)) + 128 * kk;
                        a_mma(tmem_o + (uint32_t)(64 * c), pd, vd, idesc_o, (j | kk) ? 1u : 0u);
                    }
                }
                a_commit(bar(B_PE, s));                               // the output holds tiles 0..j; V_j and P_j are free
            }
            __syncwarp();
            if (j + 2 < n_tiles) {
                if (j >= 1) ok = a_wait(bar(B_PE, (j - 1) & 1), ((j - 1) >> 1) & 1, flag);
                if (!ok) break;
                load_tile(1, j + 2);
            }
        }
        if (!ok) {
            for (int t = 0; t < 64; ++t) __nanosleep(1000);
        }
    } else if (warp >= 2) {
        // ---- softmax and output: one thread per query row -----------------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                          // row of the tile = TMEM lane
        const int q_row = tile * ABM + row;                           // index among the sequence's new tokens
        const int pos = ctx_before + q_row;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        const float scale_log2 = scale * 1.4426950408889634f;
        float used_max = -INFINITY, row_sum = 0.0f;                   // in units of log2, after the scale
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j & 1;
            const int key0 = (first_tile + j) * ABN;
            ok = a_wait(bar(B_SF, s), (j >> 1) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // a row needs masks only in tiles that reach past its own position, past the sequence's end or
            // below its window; everywhere else the raw scores are used as they are
            const bool plain = key0 + ABN - 1 <= pos && key0 + ABN - 1 < ctx && (window == 0 || key0 > pos - window);
            auto visible = [&](int key) { return key <= pos && key < ctx && (window == 0 || key > pos - window); };
            uint32_t v0[32], v1[32];                                  // the row's 64 scores
            a_ld32(tmem_s + lane_bits + (uint32_t)(64 * s), v0);
            a_ld32(tmem_s + lane_bits + (uint32_t)(64 * s + 32), v1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) a_arrive(bar(B_SE, s));                     // the scores are in registers
            float sc[ABN];
            if (plain) {
#pragma unroll
                for (int e = 0; e < 32; ++e) { sc[e] = __uint_as_float(v0[e]); sc[32 + e] = __uint_as_float(v1[e]); }
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    sc[e] = visible(key0 + e) ? __uint_as_float(v0[e]) : -INFINITY;
                    sc[32 + e] = visible(key0 + 32 + e) ? __uint_as_float(v1[e]) : -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < ABN; e += 8) {                         // (three-input maxima: two scores an instruction)
#pragma unroll
                for (int c = 0; c < 4; ++c) m4[c] = a_max3(m4[c], sc[e + 2 * c], sc[e + 2 * c + 1]);
            }
            const float tile_max = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;   // scale > 0
            // raise the maximum in use (and rescale what has been accumulated) only when it matters
            const bool raise = tile_max > used_max + RESCALE_MARGIN;
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // the output accumulator may be touched once the product of the previous tile has finished
                ok = a_wait(bar(B_PE, (j - 1) & 1), ((j - 1) >> 1) & 1, flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float corr = raise ? a_exp2(used_max - tile_max) : 1.0f;     // 0 if nothing was seen before
#pragma unroll 1
                for (int c = 0; c < AHD; c += 32) {
                    uint32_t v[32];
                    a_ld32(tmem_o + lane_bits + (uint32_t)c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                    a_st32(tmem_o + lane_bits + (uint32_t)c, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                row_sum *= corr;
            }
            if (raise) used_max = tile_max;
            const float offset = used_max == -INFINITY ? 0.0f : used_max;      // nothing visible yet: every p is 0
            // the probability buffer may be rewritten once the product two tiles back has read it
            if (j >= 2) ok = a_wait(bar(B_PE, s), ((j >> 1) - 1) & 1, flag);
            if (!ok) break;
            uint8_t* p_tile = p_ring + s * TILE_BYTES;
            float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int piece = 0; piece < ABN / 8; ++piece) {             // 8 keys = one 16-byte piece
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    // (a masked score is -infinity, the offset is finite and the scale positive: 2^-infinity = 0)
                    p[e] = a_exp2(fmaf(sc[8 * piece + e], scale_log2, -offset));
                    s4[e & 3] += p[e];
                }
                uint32_t packed[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
                    packed[e] = *(const uint32_t*)&pair;
                }
                *(uint4*)(p_tile + row * 128 + ((piece ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            row_sum += (s4[0] + s4[1]) + (s4[2] + s4[3]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) a_arrive(bar(B_PF, s));                     // probabilities in place (and any rescale done)
        }
        // the last product has finished: read the output once, normalise, store
        if (ok && n_tiles > 0) ok = a_wait(bar(B_PE, (n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, flag);
        if (ok && n_tiles > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inverse = 1.0f / row_sum;
            __nv_bfloat16* dst = out + ((size_t)(q_begin + min(q_row, q_len - 1)) * num_heads + head) * AHD;
#pragma unroll 1
            for (int c = 0; c < AHD; c += 32) {
                uint32_t v[32];
                a_ld32(tmem_o + lane_bits + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (q_row < q_len) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint32_t packed[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * e]) * inverse,
                                                                              __uint_as_float(v[d + 2 * e + 1]) * inverse);
                            packed[e] = *(const uint32_t*)&pair;
                        }
                        *(uint4*)(dst + c + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*AEncode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                            const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                            CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AEncode a_encoder() {
    static AEncode fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return (AEncode)entry;
    }();
    return fn;
}

// bfloat16 matrix [rows, cols] row-major, box of box_rows x 64 columns, 128-byte swizzle
static int a_map(const void* base, long long rows, int cols, int box_rows, CUtensorMap* out) {
    struct Key { const void* base; long long rows; int cols, box; };
    static std::mutex lock;
    static std::vector<std::pair<Key, CUtensorMap>> cache;
    std::lock_guard<std::mutex> guard(lock);
    for (auto& entry : cache)
        if (entry.first.base == base && entry.first.rows == rows && entry.first.cols == cols && entry.first.box == box_rows) {
            *out = entry.second;
            return 0;
        }
    AEncode encode = a_encoder();
    if (!encode) return fail("skv_attention_prefill_tc", "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) return fail("skv_attention_prefill_tc", "cuTensorMapEncodeTiled failed");
    if (cache.size() > 1024) cache.clear();
    cache.push_back({Key{base, rows, cols, box_rows}, map});
    *out = map;
    return 0;
}

}  // namespace skv

using namespace skv;

// As skv_attention_prefill; cache_blocks is the number of blocks of the layer's cache tensors
// [cache_blocks][kv_heads][block_size][head_dim]; n_tokens the rows of q and out.
SKV_EXPORT int skv_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, int cache_blocks,
                                        const int* block_table, int table_width, const int* cu_q,
                                        const int* ctx_after, void* out, int n_seqs, int n_tokens, int max_q_len,
                                        int num_heads, int num_kv_heads, int head_dim, int block_size, float scale,
                                        int window, int* flag, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (head_dim != AHD) return fail("skv_attention_prefill_tc", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_prefill_tc", "heads must be a positive multiple of kv heads");
    if (block_size < 16 || (block_size & (block_size - 1)) != 0)
        return fail("skv_attention_prefill_tc", "block_size must be a power of two, at least 16");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)
        return fail("skv_attention_prefill_tc", "operands must be 16-byte aligned");
    const int rows_per_load = block_size < ABN ? block_size : ABN;
    CUtensorMap map_q, map_k, map_v;
    if (int code = a_map(q, n_tokens, num_heads * AHD, 128, &map_q)) return code;
    const long long cache_rows = (long long)cache_blocks * num_kv_heads * block_size;
    if (int code = a_map(k_cache, cache_rows, AHD, rows_per_load, &map_k)) return code;
    if (int code = a_map(v_cache, cache_rows, AHD, rows_per_load, &map_v)) return code;
    const int tiles_per_seq = (max_q_len + ABM - 1) / ABM;
    const long long blocks = (long long)n_seqs * tiles_per_seq;
    if (blocks > 65535) return fail("skv_attention_prefill_tc", "too many query tiles in one step (65,535 at most)");
    const size_t smem = (size_t)(ACH + 2) * TILE_BYTES + (size_t)(K_STAGES + V_STAGES) * ACH * KV_TILE_BYTES + B_COUNT * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(prefill_attention_tc_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_attention_prefill_tc", cudaGetErrorString(status));
        configured = true;
    }
    return launch_pdl("skv_attention_prefill_tc", prefill_attention_tc_kernel, dim3(num_heads, (unsigned)blocks),
                      dim3(ATHREADS), smem, stream, map_q, map_k, map_v, block_table, table_width, cu_q, ctx_after,
                      (__nv_bfloat16*)out, num_heads, num_kv_heads, block_size, rows_per_load, scale, window,
                      tiles_per_seq, flag);
}

SKV_EXPORT int skv_has_attention_prefill_tc() { return 1; }

#else

SKV_EXPORT int skv_attention_prefill_tc(const void*, const void*, const void*, int, const int*, int, const int*,
                                        const int*, void*, int, int, int, int, int, int, int, float, int, int*,
                                        cudaStream_t) {
    return skv::fail("skv_attention_prefill_tc", "this build (float32, or a head size other than 64 or 128) has no such kernel");
}

SKV_EXPORT int skv_has_attention_prefill_tc() { return 0; }

#endif
