// Prefill GEMM on the 5th-generation tensor cores: out = A[M,K] . W[N,K]^T, bfloat16 in,
// float accumulation in tensor memory, fused epilogue (the modes of linear.cu).
//
// This is what replaces the reference's 32x32 shared-memory tile GEMM
// (src/cuda/gemm_cuda.cu:445-525) when a step brings many tokens.  At most one block per SM runs; it
// walks over 128 x BN tiles of the output with two accumulators in tensor memory, so that the epilogue
// of one tile overlaps the main loop of the next:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor) of 128x64 A and BNx64 W tiles
//            into a ring of shared-memory stages, 128-byte swizzled, completing on mbarriers;
//   warp 1   allocates 2 x BN columns of tensor memory; one thread issues tcgen05.mma
//            (128 x BN x 16 per instruction, four per stage) and commits each stage back to
//            the loader, and the finished accumulator to the epilogue;
//   warps 2-5 read the accumulator with tcgen05.ld (each warp its quarter of the 128 lanes,
//            one output row per thread), apply the epilogue into swizzled slabs of shared memory and
//            send them out with TMA stores (reduce-add for the residual).
// Tails in M, N and K are zero-filled by TMA and masked in the epilogue.
//
// Every wait on an mbarrier gives up after a bounded number of tries, raises bit 2 (value 4)
// of the caller's flag word, and lets the block drain and free its tensor memory.
#include "common.cuh"

#if SKV_DTYPE == SKV_BF16

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace skv {

enum { TC_MODE_STORE = 0, TC_MODE_STORE_F32 = 1, TC_MODE_ADD_F32 = 2, TC_MODE_GATED = 3, TC_MODE_QKV_ROPE = 4 };

// What the q|k|v projection's epilogue needs to finish the job of rope_kv_write_vec_kernel (elementwise.cu)
// itself: the output columns are [query heads | key heads | value heads]; queries and keys are rotated in float
// with the host-built table (pairs (d, d + head_dim / 2), src/layers/attention.cpp:96-135), rounded to bfloat16
// once, queries go to `q_out` (through the copy engine), keys and values of token m to row positions[m] of
// the cache block that the block table of sequence token_seq[m] names.
struct RopeArgs {
    const float2* cos_sin;             // [positions][head_dim / 2] (cos, sin), or null: no rotation
    const int* positions;              // [M]
    const int* token_seq;              // [M]
    const int* block_table;            // [sequences][table_width]
    __nv_bfloat16* k_cache;            // [blocks][kv_heads][block_size][head_dim]
    __nv_bfloat16* v_cache;
    int table_width, num_heads, num_kv_heads, head_dim, block_size, write_kv;
};

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                      // 64 bfloat16 = one 128-byte swizzle row
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Returns false if the barrier did not flip within the limit (the flag is raised then).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* flag) {
    for (uint32_t tries = 0; tries < TC_WAIT_LIMIT; ++tries) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    if (flag) atomicOr(flag, 4);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}

// out[tile] += tile, done by the copy engine in L2: nothing of `out` is read into the SM
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}

// One 16-byte piece of a thread's 128-byte output row, at its 128-byte-swizzled place in the slab
__device__ __forceinline__ void slab_write(uint8_t* slab, int row, int piece, uint4 value) {
    *(uint4*)(slab + row * 128 + ((piece ^ (row & 7)) << 4)) = value;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// start address / 16 in bits 0-13, leading offset (unused here) 1 in bits 16-29, 1024 bytes
// between 8-row groups / 16 in bits 32-45, descriptor version 1 in bits 46-47, swizzle mode 2
// (128 bytes) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: D float (1 at bit 4), A and B bfloat16 (1 at bits 7 and
// 10), both K-major (bits 15, 16 zero), N/8 at bits 17-22, M/16 at bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    return chosen != 0;
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// The gate's activation, chosen by the caller (common.cuh names them), as g * sigmoid(z) = g / (1 + e^-z): z = g for
// silu (the form of the reference's GPU kernel, src/cuda/gemm_cuda.cu:229), z = 2 sqrt(2/pi) (g + 0.044715 g^3) for the
// tanh form of gelu (g/2 (1 + tanh(z/2))).  Exponential and quotient are the special-function unit's (`ex2.approx`
// on z log2 e, `rcp.approx`): a few units in the last place of a float (2 + |1.16 z| for the exponential), far
// below the bfloat16 the product is rounded to.  With libm's expf and an IEEE division the gated epilogue of a
// 256-column tile took longer than the tile's main loop (2,048 x 11,264 x 2,048: 76.7 us against 63.8 us).  Past
// z = -88 the exponential overflows to infinity and the quotient is -0, the right limit.
__device__ __forceinline__ float gate_activation(float g, int act) {
    const float z = act == ACT_GELU_TANH ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : g;
    return __fdividef(g, 1.0f + __expf(-z));
}

// Which tile of the output a block's t-th tile is.  Row tiles run fastest, so that blocks which run together share a
// W tile; but with very many tokens the A tiles of one sweep over the rows no longer fit in L2 (39,000 tokens x 4,096
// x 2 bytes are 320 MB) and every column of tiles would fetch A from memory again.  So the rows are walked in bands:
// within a band of `band` row tiles, columns outside, rows inside; a band's A rows (at most about 40 MB, a third of
// L2: 39,294 tokens of the Llama-3-8B shape took 590 ms in one sweep, 518 / 481 / 460 / 468 / 496 ms with bands of
// 96 / 64 / 40 / 24 / 12 MB) stay in L2 while W, which is smaller, streams past once per band.
__device__ __forceinline__ void tile_coordinates(int tile, int m_tiles, int n_tiles, int band, int& m_tile, int& n_tile) {
    const int per_band = band * n_tiles;
    const int b = tile / per_band, within = tile - b * per_band;
    const int rows_here = min(band, m_tiles - b * band);
    n_tile = within / rows_here;
    m_tile = b * band + (within - n_tile * rows_here);
}

// How many row tiles of `tile_rows` rows make a band (see tile_coordinates)
__host__ __device__ inline int tile_band(int tile_rows, int K) {
    const long long bytes_per_tile = (long long)tile_rows * K * 2;
    const long long band = (40ll << 20) / (bytes_per_tile > 0 ? bytes_per_tile : 1);
    return (int)(band < 1 ? 1 : (band > (1 << 20) ? (1 << 20) : band));
}

// The epilogue of one output tile for one of the four epilogue warps: reads the warp's quarter of the
// accumulator (TMEM lanes 32*quarter .., one output row per thread) and stores it in the mode asked for.
template <int BN>
__device__ __forceinline__ void epilogue_tile(uint32_t acc_tmem, int quarter, int lane, uint8_t* slabs, int& buffer,
                                              const CUtensorMap* map_out, int tma_out, void* __restrict__ out, int M,
                                              int N, int mode, int act, int m0, int n0) {
    const int m = m0 + quarter * 32 + lane;
    if (tma_out) {
        // Each thread builds 128 bytes of its output row in a swizzled slab of shared memory; one lane
        // hands the warp's 32 x 128-byte slab to the copy engine, which writes whole rows (or adds them,
        // for the residual) and clips at M and N.
        // Two slabs per warp alternate so that one is written while the other is being read.
        const uint32_t lane_base = acc_tmem + ((uint32_t)(quarter * 32) << 16);
        const int y = m0 + quarter * 32;
        // accumulator columns that make one 128-byte output row, and output columns per slab
        const int acc_per_slab = mode == TC_MODE_GATED ? 128 : (mode == TC_MODE_STORE ? 64 : 32);
        const int out_per_slab = mode == TC_MODE_STORE_F32 || mode == TC_MODE_ADD_F32 ? 32 : 64;
        const int out_x0 = mode == TC_MODE_GATED ? (n0 >> 1) : n0;
#pragma unroll 1
        for (int seg = 0; seg * acc_per_slab < BN; ++seg) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            uint8_t* slab = slabs + buffer * 4096;
#pragma unroll 1
            for (int sub = 0; sub * 32 < acc_per_slab; ++sub) {
                uint32_t v[32];
                tmem_load_32(lane_base + (uint32_t)(seg * acc_per_slab + sub * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (mode == TC_MODE_GATED) {
                    // 32 accumulator columns = two groups of (8 gate, 8 up) -> 16 outputs = 2 pieces
#pragma unroll
                    for (int grp = 0; grp < 2; ++grp) {
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float lo = gate_activation(__uint_as_float(v[16 * grp + 2 * j]), act) *
                                             __uint_as_float(v[16 * grp + 8 + 2 * j]);
                            const float hi = gate_activation(__uint_as_float(v[16 * grp + 2 * j + 1]), act) *
                                             __uint_as_float(v[16 * grp + 8 + 2 * j + 1]);
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                            packed[j] = *(const uint32_t*)&pair;
                        }
                        slab_write(slab, lane, sub * 2 + grp, make_uint4(packed[0], packed[1], packed[2], packed[3]));
                    }
                } else if (mode == TC_MODE_STORE) {
#pragma unroll
                    for (int piece = 0; piece < 4; ++piece) {
                        uint32_t packed[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(
                                __uint_as_float(v[8 * piece + 2 * e]), __uint_as_float(v[8 * piece + 2 * e + 1]));
                            packed[e] = *(const uint32_t*)&pair;
                        }
                        slab_write(slab, lane, sub * 4 + piece, make_uint4(packed[0], packed[1], packed[2], packed[3]));
                    }
                } else {
#pragma unroll
                    for (int piece = 0; piece < 8; ++piece)
                        slab_write(slab, lane, piece, make_uint4(v[4 * piece], v[4 * piece + 1], v[4 * piece + 2], v[4 * piece + 3]));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                const int x = out_x0 + seg * out_per_slab;
                const int out_cols = mode == TC_MODE_GATED ? (N >> 1) : N;
                if (x < out_cols && y < M) {             // a slab wholly outside the matrix is not sent
                    if (mode == TC_MODE_ADD_F32) tma_reduce_add_2d(map_out, x, y, smem_addr(slab));
                    else tma_store_2d(map_out, x, y, smem_addr(slab));
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            buffer ^= 1;
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
            uint32_t v[32];
            tmem_load_32(acc_tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (m >= M) continue;
            const int n = n0 + c;
            if (mode == TC_MODE_GATED) {
                // columns come in groups of 16: 8 gate columns, then their 8 up columns
                const int half_n = N >> 1;
                __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)m * half_n + (n >> 1);
#pragma unroll
                for (int grp = 0; grp < 2; ++grp) {
                    if (n + 16 * grp < N) {
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float lo = gate_activation(__uint_as_float(v[16 * grp + 2 * j]), act) *
                                             __uint_as_float(v[16 * grp + 8 + 2 * j]);
                            const float hi = gate_activation(__uint_as_float(v[16 * grp + 2 * j + 1]), act) *
                                             __uint_as_float(v[16 * grp + 8 + 2 * j + 1]);
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                            packed[j] = *(const uint32_t*)&pair;
                        }
                        *(uint4*)(dst + 8 * grp) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                }
            } else if (mode == TC_MODE_STORE) {
                __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)m * N + n;
                if (n + 32 <= N && (N & 7) == 0) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint32_t packed[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * e]),
                                                                              __uint_as_float(v[j + 2 * e + 1]));
                            packed[e] = *(const uint32_t*)&pair;
                        }
                        *(uint4*)(dst + j) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                } else {
                    for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
                }
            } else {
                float* dst = (float*)out + (size_t)m * N + n;
                const bool add = mode == TC_MODE_ADD_F32;
                if (n + 32 <= N && (N & 3) == 0) {
                    // all old values are fetched before anything is stored: a store between two
                    // loads of the same array would make each load wait for the one before
                    float4 old[8];
                    if (add) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) old[j] = __ldcg((const float4*)(dst + 4 * j));
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) old[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 r = old[j];
                        r.x += __uint_as_float(v[4 * j]); r.y += __uint_as_float(v[4 * j + 1]);
                        r.z += __uint_as_float(v[4 * j + 2]); r.w += __uint_as_float(v[4 * j + 3]);
                        *(float4*)(dst + 4 * j) = r;
                    }
                } else {
                    for (int j = 0; j < 32 && n + j < N; ++j)
                        dst[j] = (add ? dst[j] : 0.0f) + __uint_as_float(v[j]);
                }
            }
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&pair;
}

// The epilogue of one tile of the q|k|v projection with the rotary encoding and the cache write folded in
// (TC_MODE_QKV_ROPE; head size 64 or 128, which divide the tile's width).  A thread owns a token (a row of the
// accumulator); head by head it reads 32 pairs (d, d + half) at a time, rotates them and rounds them.  A query
// head's row goes into the warp's swizzled slabs (64 columns each) and out through the copy engine; key and
// value rows are few (the KV heads) and go straight to their cache rows in 16-byte pieces.
template <int BN>
__device__ __forceinline__ void epilogue_tile_rope(uint32_t acc_tmem, int quarter, int lane, uint8_t* slabs, int& buffer,
                                                   const CUtensorMap* map_q, const RopeArgs& rope, int M, int N, int m0,
                                                   int n0) {
    const int m = m0 + quarter * 32 + lane;
    const bool row_live = m < M;
    const int hd = rope.head_dim, half = hd >> 1, n_slabs = hd >> 6;
    const uint32_t lane_base = acc_tmem + ((uint32_t)(quarter * 32) << 16);
    const int y = m0 + quarter * 32;
    const int pos = row_live ? rope.positions[m] : 0;
    size_t cache_row = 0;                          // element offset of this token's row in KV head 0 of its block
    if (row_live && rope.write_kv) {
        const int block = rope.block_table[(size_t)rope.token_seq[m] * rope.table_width + pos / rope.block_size];
        cache_row = ((size_t)block * rope.num_kv_heads * rope.block_size + (pos % rope.block_size)) * hd;
    }
    const float4* angles = rope.cos_sin ? (const float4*)(rope.cos_sin + (size_t)pos * half) : nullptr;
#pragma unroll 1
    for (int col0 = 0; col0 < BN && n0 + col0 < N; col0 += hd) {
        const int head = (n0 + col0) / hd;
        const int kind = head < rope.num_heads ? 0 : (head < rope.num_heads + rope.num_kv_heads ? 1 : 2);
        if (kind != 0 && !rope.write_kv) continue;                  // a layer that only reads a cache another one wrote
        if (kind == 2) {
            __nv_bfloat16* dst = rope.v_cache + cache_row + (size_t)(head - rope.num_heads - rope.num_kv_heads) * rope.block_size * hd;
#pragma unroll 1
            for (int c = 0; c < hd; c += 32) {
                uint32_t v[32];
                tmem_load_32(lane_base + (uint32_t)(col0 + c), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_live) {
#pragma unroll
                    for (int piece = 0; piece < 4; ++piece)
                        *(uint4*)(dst + c + 8 * piece) = make_uint4(
                            pack_bf16(__uint_as_float(v[8 * piece]), __uint_as_float(v[8 * piece + 1])),
                            pack_bf16(__uint_as_float(v[8 * piece + 2]), __uint_as_float(v[8 * piece + 3])),
                            pack_bf16(__uint_as_float(v[8 * piece + 4]), __uint_as_float(v[8 * piece + 5])),
                            pack_bf16(__uint_as_float(v[8 * piece + 6]), __uint_as_float(v[8 * piece + 7])));
                }
            }
            continue;
        }
        uint8_t* slab0 = slabs;                    // a query head's row: one slab (head size 64) or both (128)
        if (kind == 0) {
            if (n_slabs == 1) {                    // the two slabs alternate: one is written while the other is being read
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                slab0 = slabs + buffer * 4096;
            } else {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
            __syncwarp();
        }
        __nv_bfloat16* key_dst = rope.k_cache + cache_row + (size_t)(head - rope.num_heads) * rope.block_size * hd;
#pragma unroll 1
        for (int c = 0; c < half; c += 32) {       // pairs c .. c + 31
            uint32_t lo[32], hi[32];
            tmem_load_32(lane_base + (uint32_t)(col0 + c), lo);
            tmem_load_32(lane_base + (uint32_t)(col0 + half + c), hi);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int piece = 0; piece < 4; ++piece) {                // eight pairs: one 16-byte piece of each half
                uint32_t first[4], second[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {                        // two pairs at a time
                    float4 cs = make_float4(1.0f, 0.0f, 1.0f, 0.0f);  // (cos, sin) of pairs 2e and 2e + 1 of the piece
                    if (angles) cs = angles[(c + 8 * piece + 2 * e) >> 1];
                    const float a0 = __uint_as_float(lo[8 * piece + 2 * e]), a1 = __uint_as_float(lo[8 * piece + 2 * e + 1]);
                    const float b0 = __uint_as_float(hi[8 * piece + 2 * e]), b1 = __uint_as_float(hi[8 * piece + 2 * e + 1]);
                    first[e] = pack_bf16(a0 * cs.x - b0 * cs.y, a1 * cs.z - b1 * cs.w);      // as rotated() of elementwise.cu
                    second[e] = pack_bf16(a0 * cs.y + b0 * cs.x, a1 * cs.w + b1 * cs.z);
                }
                const uint4 low = make_uint4(first[0], first[1], first[2], first[3]);
                const uint4 high = make_uint4(second[0], second[1], second[2], second[3]);
                const int d_low = c + 8 * piece, d_high = half + c + 8 * piece;      // element of the head's row
                if (kind == 0) {
                    slab_write(slab0 + (d_low >> 6) * 4096, lane, (d_low & 63) >> 3, low);
                    slab_write(slab0 + (d_high >> 6) * 4096, lane, (d_high & 63) >> 3, high);
                } else if (row_live) {
                    *(uint4*)(key_dst + d_low) = low;
                    *(uint4*)(key_dst + d_high) = high;
                }
            }
        }
        if (kind == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if (y < M) {
                    for (int sl = 0; sl < n_slabs; ++sl)
                        tma_store_2d(map_q, head * hd + sl * 64, y, smem_addr(slab0 + sl * 4096));
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (n_slabs == 1) buffer ^= 1;
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, int tma_out, void* __restrict__ out, int M,
                    int N, int K, int mode, int act, int* __restrict__ flag, const RopeArgs rope) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    // tensor memory is handed out in powers of two columns: two accumulators, each at the start of a half
    constexpr uint32_t TMEM_COLS = BN <= 64 ? 128 : (BN <= 128 ? 256 : 512), ACC_STRIDE = TMEM_COLS / 2;
    static_assert(BN % 32 == 0 && BN <= 256 && STAGE_BYTES % 1024 == 0, "tile width");
    constexpr uint32_t SLAB_BYTES = 4 * 2 * 4096;           // four epilogue warps, two 32 x 128-byte slabs each
    extern __shared__ uint8_t smem_raw[];
    // tiles and slabs need 1024-byte alignment for the 128-byte swizzle
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* slab_base = tiles + (size_t)STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(slab_base + SLAB_BYTES);   // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int band = tile_band(TC_BM, K);
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
    const uint32_t acc_full0 = smem_addr(bars + 2 * STAGES), acc_empty0 = smem_addr(bars + 2 * STAGES + 2);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // two accumulators of BN columns each: the epilogue of one tile overlaps the main loop of the next
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                   // A is the previous kernel's output

    // A block walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...; neighbouring tiles share their
    // W rows (m runs fastest), so blocks that run together read the same W tile from L2.
    if (warp == 0) {
        // ---- loader: the whole warp walks the loop, one elected lane issues ------------------------
        bool ok = true;
        int it = 0;                               // k iterations issued so far, over all tiles
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            int m_tile, n_tile;
            tile_coordinates(tile, m_tiles, n_tiles, band, m_tile, n_tile);
            const int m0 = m_tile * TC_BM, n0 = n_tile * BN;
            for (int i = 0; i < k_iters; ++i, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, flag);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, i * TC_BK, m0, full0 + 8 * s);
                    tma_load_2d(a_dst + A_BYTES, &map_w, i * TC_BK, n0, full0 + 8 * s);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            // let the copies in flight land before the block leaves (bounded)
            for (int i = max(0, it - STAGES); i < it; ++i) mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr);
        }
    } else if (warp == 1) {
        // ---- tensor-core issue: the whole warp walks the loop, one elected lane issues ----------------
        constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
        bool ok = true;
        int it = 0, local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            if (local >= 2) {                     // the epilogue must have drained this accumulator
                ok = mbar_wait(acc_empty0 + 8 * buf, ((local >> 1) - 1) & 1, flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            const uint32_t acc = tmem_base + (uint32_t)buf * ACC_STRIDE;
            for (int i = 0; i < k_iters; ++i, ++it) {
                const int s = it % STAGES;
                ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
                    const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc(a_addr), w_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        // 16 bfloat16 = 32 bytes further along K: +2 in the descriptor's 16-byte units
                        umma_bf16(acc, a_desc + 2 * k, w_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);  // frees the stage when these MMAs have read it
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit(acc_full0 + 8 * buf);   // arrives when every MMA of the tile has finished
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ---- epilogue ---------------------------------------------------------------------------
        const int quarter = warp & 3;             // the TMEM lanes this warp may read
        uint8_t* slabs = slab_base + quarter * 8192;
        int buffer = 0, local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            ok = mbar_wait(acc_full0 + 8 * buf, (local >> 1) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int m_tile, n_tile;
            tile_coordinates(tile, m_tiles, n_tiles, band, m_tile, n_tile);
            const int m0 = m_tile * TC_BM, n0 = n_tile * BN;
            if (mode == TC_MODE_QKV_ROPE) {
                if constexpr (BN % 128 == 0)
                    epilogue_tile_rope<BN>(tmem_base + (uint32_t)buf * ACC_STRIDE, quarter, lane, slabs, buffer, &map_out, rope,
                                           M, N, m0, n0);
            } else {
                epilogue_tile<BN>(tmem_base + (uint32_t)buf * ACC_STRIDE, quarter, lane, slabs, buffer, &map_out, tma_out, out,
                                  M, N, mode, act, m0, n0);
            }
            // the accumulator has been read out: hand it back to the issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
        }
        if (tma_out) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- pairs of blocks: one 256 x 256 tile per two SMs ------------------------------------------------
// A block of the kernel above has to fetch 48 KB (128 rows of A and 256 of W, 64 wide) for 512 cycles of tensor
// work, 96 bytes a cycle, and an SM takes in about 64: its tensor pipe measured busy two thirds of the time.  Here
// two blocks of a cluster share a tile of 256 x 256: each fetches its 128 rows of A and its half (128 rows) of W,
// 32 KB for the same 512 cycles, and one thread of the first block issues tcgen05.mma.cta_group::2, which reads both
// halves of W from the two blocks' shared memory and leaves each block its 128 rows of the result in its own
// tensor memory.  The copies of both blocks complete on the first block's barriers (it expects the bytes of
// both); a commit frees a stage, or hands over an accumulator, in both blocks at once; the epilogue warps of both
// blocks return an accumulator to the first block's issuer.  The epilogue itself is the one of the kernel above.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

// The address, in the cluster's shared window, of what lies at `addr` in block `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_address(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}

// A copy into this block's shared memory whose bytes count on a barrier of the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t first_block_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(first_block_bar)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives, when the MMAs issued so far have finished, on the barrier at this offset in both blocks of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}

// (Tried: stages of two chunks of 64 columns, each operand brought by one copy of 32 KB through a three-dimensional
// tensor map as in the few-token kernel below, three stages.  The layer shapes did not move, 65.7 against 66.5 us for
// 2,048 x 11,264 x 2,048; 8,192 cubed went from 799 to 760 us.  Copies from L2 come back soon enough for three of 16 KB
// on their way to feed the tensor pipe.)
template <int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_out, int tma_out, void* __restrict__ out, int M,
                         int N, int K, int mode, int act, int* __restrict__ flag, const RopeArgs rope) {
    constexpr int BN = 256;                                  // the pair's tile: 256 rows (128 per block) x 256 columns
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, W_BYTES = (BN / 2) * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr uint32_t TMEM_COLS = 512, ACC_STRIDE = 256;
    constexpr uint32_t SLAB_BYTES = 4 * 2 * 4096;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* slab_base = tiles + (size_t)STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(slab_base + SLAB_BYTES);   // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                   // 0: the block that issues the pair's MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (M + 2 * TC_BM - 1) / (2 * TC_BM), n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int band = tile_band(2 * TC_BM, K);
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
    const uint32_t acc_full0 = smem_addr(bars + 2 * STAGES), acc_empty0 = smem_addr(bars + 2 * STAGES + 2);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        // full and acc_empty are used in the first block only: one arrival (its loader's, with the bytes of both
        // blocks) and one per epilogue warp of both blocks
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    // both blocks' barriers exist before either signals the other's
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        // ---- loader: this block's rows of A and its half of the W rows (the warp walks, an elected lane issues) ----
        bool ok = true;
        int it = 0;
        const uint32_t first_full0 = cluster_address(full0, 0);
        for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
            int m_tile, n_tile;
            tile_coordinates(tile, m_tiles, n_tiles, band, m_tile, n_tile);
            const int m0 = m_tile * 2 * TC_BM + (int)rank * TC_BM;
            const int w0 = n_tile * BN + (int)rank * (BN / 2);
            for (int i = 0; i < k_iters; ++i, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, flag);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &map_a, i * TC_BK, m0, first_full0 + 8 * s);
                    tma_load_2d_pair(a_dst + A_BYTES, &map_w, i * TC_BK, w0, first_full0 + 8 * s);
                }
                __syncwarp();
            }
        }
        if (!ok && rank == 0) {
            // let the copies in flight land before the pair leaves (bounded); the other block waits for this
            // one at the cluster barrier below
            for (int i = max(0, it - STAGES); i < it; ++i) mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr);
        }
    } else if (warp == 1 && rank == 0) {
        // ---- tensor-core issue, for both blocks: the warp walks the loop, one elected lane issues -----
        constexpr uint32_t idesc = umma_idesc(2 * TC_BM, BN);
        bool ok = true;
        int it = 0, local = 0;
        for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
            const int buf = local & 1;
            if (local >= 2) {
                ok = mbar_wait(acc_empty0 + 8 * buf, ((local >> 1) - 1) & 1, flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            const uint32_t acc = tmem_base + (uint32_t)buf * ACC_STRIDE;
            for (int i = 0; i < k_iters; ++i, ++it) {
                const int s = it % STAGES;
                ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
                    const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc(a_addr), w_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(acc, a_desc + 2 * k, w_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty0 + 8 * s);
                }
                __syncwarp();
            }
            if (ok && elect_one()) umma_commit_pair(acc_full0 + 8 * buf);
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ---- epilogue: this block's 128 rows of the tile ------------------------------------------
        const int quarter = warp & 3;
        uint8_t* slabs = slab_base + quarter * 8192;
        int buffer = 0, local = 0;
        bool ok = true;
        const uint32_t first_acc_empty0 = cluster_address(acc_empty0, 0);
        for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
            const int buf = local & 1;
            ok = mbar_wait(acc_full0 + 8 * buf, (local >> 1) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int m_tile, n_tile;
            tile_coordinates(tile, m_tiles, n_tiles, band, m_tile, n_tile);
            const int m0 = m_tile * 2 * TC_BM + (int)rank * TC_BM, n0 = n_tile * BN;
            if (mode == TC_MODE_QKV_ROPE) {
                epilogue_tile_rope<BN>(tmem_base + (uint32_t)buf * ACC_STRIDE, quarter, lane, slabs, buffer, &map_out, rope,
                                       M, N, m0, n0);
            } else {
                epilogue_tile<BN>(tmem_base + (uint32_t)buf * ACC_STRIDE, quarter, lane, slabs, buffer, &map_out, tma_out, out,
                                  M, N, mode, act, m0, n0);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];"
                             ::"r"(first_acc_empty0 + 8 * buf) : "memory");
        }
        if (tma_out) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __syncwarp();
        }
    }
    // neither block leaves, or frees its tensor memory, while the other may still read its shared memory or
    // signal its barriers
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- few tokens: the weights take the 128 rows of the instruction ---------------------------------
// For steps of 17 to 128 tokens the tile above would use a fraction of its 128 token rows and leave most SMs
// without a tile.  Here the operands change places: D^T[128 weight rows, tokens] = W_tile . X^T, so a block
// owns 128 rows of W (all of K, or one of `splits` parts of it) and every token; the grid has N/128 x splits
// blocks that stream their weights once, through a deep ring, with the first stages requested before the
// wait on the kernel in front (weights do not depend on it).  In the epilogue a thread holds one weight
// row's results for 32 tokens at a time, and the 32 lanes of a warp write 32 neighbouring columns of a
// token's output row.  With splits > 1 the blocks of a cluster each take a part of K; the others push their
// accumulators into the first block's shared memory, which adds them in rank order.
// A stage holds CH chunks of 64 columns.  With CH = 2 one copy brings both chunks of the weight rows (and one those of the
// tokens): the tensor maps are then three-dimensional, [64][rows][K / 64] with the chunk index as the slowest dimension of
// the box, and the box lands as CH tiles of rows x 64, one behind the other.  An SM keeps only about three copies on their
// way whatever their size, so copies of 16 KB stream 45 GB/s into a block and copies of 32 KB 65 (88 blocks: 3.6
// against 4.5 TB/s over the GPU).  That form needs K to be a multiple of 64 (a chunk that K cuts would continue into the
// next row); other K take CH = 1 with the two-dimensional maps, which fill the tail with zeros.
template <int MP, int STAGES, int CH>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_few_tokens_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                               void* __restrict__ out, int M, int N, int K, int mode, int act, int splits,
                               int* __restrict__ flag) {
    constexpr uint32_t W_CHUNK = 128 * TC_BK * 2, X_CHUNK = MP * TC_BK * 2;
    constexpr uint32_t W_BYTES = W_CHUNK * CH, X_BYTES = X_CHUNK * CH, STAGE_BYTES = W_BYTES + X_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + (size_t)STAGES * STAGE_BYTES);      // full[STAGES], empty[STAGES], acc_full
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 128;
    const int split = blockIdx.y;                                           // == rank in the cluster
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int per_split = (k_blocks + splits - 1) / splits;
    const int k_first = split * per_split, my_chunks = max(0, min(k_blocks, k_first + per_split) - k_first);
    const int k_iters = (my_chunks + CH - 1) / CH;                          // stages of CH chunks (the last may hold fewer)
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES), acc_full = smem_addr(bars + 2 * STAGES);
    auto load_w = [&](uint32_t dst, int i, uint32_t bar) {
        if (CH == 1) tma_load_2d(dst, &map_w, (k_first + i) * TC_BK, n0, bar);
        else tma_load_3d(dst, &map_w, 0, n0, k_first + i * CH, bar);
    };
    auto load_x = [&](uint32_t dst, int i, uint32_t bar) {
        if (CH == 1) tma_load_2d(dst, &map_x, (k_first + i) * TC_BK, 0, bar);
        else tma_load_3d(dst, &map_x, 0, 0, k_first + i * CH, bar);
    };

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)MP) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- loader: weights of the first stages before the wait, activations after it ----------------
        bool ok = true;
        const int ahead = min(STAGES, k_iters);
        for (int i = 0; i < ahead; ++i) {
            mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
            load_w(smem_addr(tiles + (size_t)i * STAGE_BYTES), i, full0 + 8 * i);
        }
        pdl_wait();
        for (int i = 0; i < ahead; ++i) load_x(smem_addr(tiles + (size_t)i * STAGE_BYTES) + W_BYTES, i, full0 + 8 * i);
        for (int i = ahead; i < k_iters && ok; ++i) {
            const int s = i % STAGES;
            ok = mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, flag);
            if (!ok) break;
            const uint32_t dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
            mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
            load_w(dst, i, full0 + 8 * s);
            load_x(dst + W_BYTES, i, full0 + 8 * s);
        }
        if (!ok) {
            for (int i = max(0, k_iters - STAGES); i < k_iters; ++i) mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr);
        }
    } else if (warp == 1) {
        // ---- tensor-core issue: the warp walks the loop whole and one elected lane issues (a lone lane under
        // `lane == 0` took about 95 cycles per tcgen05 instruction in the prefill attention kernel, an elected
        // lane of a converged warp 70; with eight small stages a block that chain is on the kernel's path) -------
        constexpr uint32_t idesc = umma_idesc(128, MP);
        bool ok = true;
        for (int i = 0; i < k_iters && ok; ++i) {
            const int s = i % STAGES;
            ok = mbar_wait(full0 + 8 * s, (i / STAGES) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (elect_one()) {
                const uint32_t w_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    // (a stage's second chunk may lie past this block's part of K: it was copied, it is not used)
                    if (i * CH + c < my_chunks) {
                        const uint64_t w_desc = umma_desc(w_addr + c * W_CHUNK), x_desc = umma_desc(w_addr + W_BYTES + c * X_CHUNK);
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)
                            umma_bf16(tmem_base, w_desc + 2 * k, x_desc + 2 * k, idesc, (i > 0 || c > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(empty0 + 8 * s);
            }
            __syncwarp();
        }
        if (ok && elect_one()) umma_commit(acc_full);   // arrives when every MMA has finished (at once if there were none)
        __syncwarp();
    }
    // ---- epilogue: warps 2-5, one weight row per thread -----------------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // weight row within the tile = TMEM lane
    const int n = n0 + row;
    bool ok = true;
    // In the residual-add mode the first 64 tokens' old values are fetched while the main loop runs.
    constexpr int EARLY = MP < 64 ? MP : 64;
    float early[EARLY];
    if (warp >= 2) {
        pdl_wait();                               // the residual stream that the epilogue reads is the kernels' before
        if (mode == TC_MODE_ADD_F32 && split == 0) {
#pragma unroll
            for (int j = 0; j < EARLY; ++j)
                early[j] = (j < M && n < N) ? __ldcg((const float*)out + (size_t)j * N + n) : 0.0f;
        }
        ok = k_iters == 0 || mbar_wait(acc_full, 0, flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    auto read_accumulator = [&](int c, uint32_t (&v)[32]) {
        if (ok && k_iters > 0) {
            tmem_load_32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
    };
    // With splits, the partial results [tokens][128 rows] of ranks 1.. go to rank 0's shared memory, where the
    // pipeline's stages lay: the first cluster barrier is passed when every block's main loop is over (the
    // epilogue warps get there after their accumulator is complete), the second when the pushes are done.
    float* inbox = (float*)tiles;                 // [splits - 1][MP][128] floats, in rank 0
    if (splits > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (split > 0 && warp >= 2) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(inbox)), "r"(0));
            remote += (uint32_t)(split - 1) * MP * 128 * 4;
#pragma unroll 1
            for (int c = 0; c < MP && c < M; c += 32) {
                uint32_t v[32];
                read_accumulator(c, v);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + (uint32_t)((c + j) * 128 + row) * 4), "r"(v[j]) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp >= 2 && split == 0) {
#pragma unroll
        for (int c = 0; c < MP; c += 32) {
            if (c >= M) break;
            uint32_t v[32];
            read_accumulator(c, v);
            for (int r = 1; r < splits; ++r) {    // rank order: the sum does not depend on timing
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    v[j] = __float_as_uint(__uint_as_float(v[j]) + inbox[((size_t)(r - 1) * MP + c + j) * 128 + row]);
            }
            if (mode == TC_MODE_GATED) {
                // rows come in groups of 16: 8 gate rows, then their 8 up rows; lane l < 8 (mod 16) pairs with l + 8
                const int half_n = N >> 1;
                const int o = ((n >> 4) << 3) + (n & 7);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float up = __shfl_down_sync(0xffffffffu, __uint_as_float(v[j]), 8);
                    if ((lane & 8) == 0 && c + j < M && n < N)
                        ((__nv_bfloat16*)out)[(size_t)(c + j) * half_n + o] =
                            __float2bfloat16_rn(gate_activation(__uint_as_float(v[j]), act) * up);
                }
            } else if (n < N) {
                if (mode == TC_MODE_STORE) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c + j < M) ((__nv_bfloat16*)out)[(size_t)(c + j) * N + n] = __float2bfloat16_rn(__uint_as_float(v[j]));
                } else if (mode == TC_MODE_STORE_F32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c + j < M) ((float*)out)[(size_t)(c + j) * N + n] = __uint_as_float(v[j]);
                } else {
                    float old[32];
                    if (c < EARLY) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) old[j] = early[(c < EARLY ? c : 0) + j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) old[j] = c + j < M ? __ldcg((const float*)out + (size_t)(c + j) * N + n) : 0.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c + j < M) ((float*)out)[(size_t)(c + j) * N + n] = old[j] + __uint_as_float(v[j]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)MP) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return (EncodeTiled)entry;
    }();
    return fn;
}

struct MapKey {
    const void* base; int rows, cols, box_rows, box_cols, elem_bytes;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows &&
               box_cols == o.box_cols && elem_bytes == o.elem_bytes;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.cols << 21) ^
               ((size_t)k.box_rows << 7) ^ ((size_t)k.box_cols << 3) ^ (size_t)k.elem_bytes;
    }
};

// A row-major [rows, cols] matrix of bfloat16 (elem_bytes 2) or float (4), box of box_rows x box_cols
// elements whose rows are at most 128 bytes, 128-byte swizzle.
static int tensor_map(const void* base, int rows, int cols, int elem_bytes, int box_rows, int box_cols,
                      CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, cols, box_rows, box_cols, elem_bytes};
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(key);
    if (found != cache.end()) { *out = found->second; return 0; }
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail("skv_linear(tcgen05)", "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult status = encode(&map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                   2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        char detail[64];
        snprintf(detail, sizeof detail, "cuTensorMapEncodeTiled failed with code %d", (int)status);
        return fail("skv_linear(tcgen05)", detail);
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return 0;
}

// A bfloat16 matrix [rows, K], K a multiple of 64, seen as [64][rows][K / 64]: a box of 64 x box_rows x chunks brings
// `chunks` neighbouring tiles of box_rows x 64 in one copy, tile after tile in shared memory (each 128-byte swizzled as
// the two-dimensional map leaves it).  Rows past the matrix and chunks past K are filled with zeros.
static int tensor_map_chunks(const void* base, int rows, int K, int box_rows, int chunks, CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, K, box_rows, -chunks, 2};
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(key);
    if (found != cache.end()) { *out = found->second; return 0; }
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail("skv_linear(tcgen05)", "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {(cuuint64_t)TC_BK, (cuuint64_t)rows, (cuuint64_t)(K / TC_BK)};
    const cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)TC_BK * 2};
    const cuuint32_t box[3] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows, (cuuint32_t)chunks};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap map;
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        char detail[64];
        snprintf(detail, sizeof detail, "cuTensorMapEncodeTiled (chunks) failed with code %d", (int)status);
        return fail("skv_linear(tcgen05)", detail);
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return 0;
}

static int tc_sm_count() { return sm_count(); }

template <int BN, int STAGES>
static int launch_tc(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act, int* flag,
                     cudaStream_t stream, const RopeArgs& rope = RopeArgs{}) {
    CUtensorMap map_a, map_w, map_out;
    if (int code = tensor_map(a, M, K, 2, TC_BM, TC_BK, &map_a)) return code;
    if (int code = tensor_map(w, N, K, 2, BN, TC_BK, &map_w)) return code;
    // The epilogue stores through the copy engine when the output's rows are 16-byte multiples;
    // otherwise (an odd vocabulary, say) the threads store their rows themselves.
    const bool float_out = mode == TC_MODE_STORE_F32 || mode == TC_MODE_ADD_F32;
    // (with the rotary epilogue `out` is the queries' tensor, [M, heads x head size] bfloat16)
    const int out_cols = mode == TC_MODE_GATED ? N / 2 : (mode == TC_MODE_QKV_ROPE ? rope.num_heads * rope.head_dim : N);
    const int out_elem = float_out ? 4 : 2;
    int tma_out = ((size_t)out_cols * out_elem) % 16 == 0 && ((uintptr_t)out & 15) == 0 ? 1 : 0;
    if (mode == TC_MODE_QKV_ROPE && !tma_out) return fail("skv_linear_qkv_rope", "the queries' rows must be 16-byte multiples");
    if (tma_out) {
        if (int code = tensor_map(out, M, out_cols, out_elem, 32, float_out ? 32 : 64, &map_out)) return code;
    } else {
        map_out = map_a;
    }
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 4 * 2 * 4096 +
                            (2 * STAGES + 4) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_linear(tcgen05)", cudaGetErrorString(status));
        configured = true;
    }
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0)
            return fail("skv_linear(tcgen05)", "cannot read the number of SMs");
    }
    const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
    dim3 grid((unsigned)(tiles < sm_count ? tiles : sm_count));     // one persistent block per SM at most
    return launch_pdl("skv_linear(tcgen05)", gemm_tcgen05_kernel<BN, STAGES>, grid, dim3(TC_THREADS), smem, stream,
                      map_a, map_w, map_out, tma_out, out, M, N, K, mode, act, flag, rope);
}

// The two-block form: clusters of two blocks, as many as the GPU runs at once (74 on 148 SMs), walk the 256 x 256 tiles.
constexpr int PAIR_STAGES = 6;
constexpr size_t PAIR_SMEM = (size_t)PAIR_STAGES * (TC_BM * TC_BK * 2 + 128 * TC_BK * 2) + 4 * 2 * 4096 +
                             (2 * PAIR_STAGES + 4) * 8 + 16 + 1024;

static void pair_launch_config(cudaLaunchConfig_t* config, cudaLaunchAttribute* attributes, cudaStream_t stream) {
    *config = cudaLaunchConfig_t{};
    config->blockDim = dim3(TC_THREADS);
    config->dynamicSmemBytes = PAIR_SMEM;
    config->stream = stream;
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config->attrs = attributes;
    config->numAttrs = 1;
}

// How many pairs of blocks the GPU runs at once (0: this GPU cannot run the two-block kernel; it is not used then)
static int pair_slots() {
    static int slots = -1;
    if (slots < 0) {
        slots = 0;
        cudaLaunchConfig_t config;
        cudaLaunchAttribute attributes[2];
        pair_launch_config(&config, attributes, nullptr);
        config.gridDim = dim3((unsigned)(tc_sm_count() / 2 * 2));
        int clusters = 0;
        if (tc_sm_count() >= 2 &&
            cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<PAIR_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)PAIR_SMEM) == cudaSuccess &&
            cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<PAIR_STAGES>, &config) == cudaSuccess && clusters > 0)
            slots = clusters < tc_sm_count() / 2 ? clusters : tc_sm_count() / 2;
        else
            cudaGetLastError();                    // (the refusal is an answer, not an error of the caller's)
    }
    return slots;
}

static int launch_pair(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act, int* flag,
                       cudaStream_t stream, const RopeArgs& rope = RopeArgs{}) {
    CUtensorMap map_a, map_w, map_out;
    if (int code = tensor_map(a, M, K, 2, TC_BM, TC_BK, &map_a)) return code;
    if (int code = tensor_map(w, N, K, 2, 128, TC_BK, &map_w)) return code;
    const bool float_out = mode == TC_MODE_STORE_F32 || mode == TC_MODE_ADD_F32;
    const int out_cols = mode == TC_MODE_GATED ? N / 2 : (mode == TC_MODE_QKV_ROPE ? rope.num_heads * rope.head_dim : N);
    const int out_elem = float_out ? 4 : 2;
    int tma_out = ((size_t)out_cols * out_elem) % 16 == 0 && ((uintptr_t)out & 15) == 0 ? 1 : 0;
    if (mode == TC_MODE_QKV_ROPE && !tma_out) return fail("skv_linear_qkv_rope", "the queries' rows must be 16-byte multiples");
    if (tma_out) {
        if (int code = tensor_map(out, M, out_cols, out_elem, 32, float_out ? 32 : 64, &map_out)) return code;
    } else {
        map_out = map_a;
    }
    const int slots = pair_slots();
    if (slots <= 0) return fail("skv_linear(tcgen05 pair)", "this GPU runs no cluster of two such blocks");
    cudaLaunchConfig_t config;
    cudaLaunchAttribute attributes[2];
    pair_launch_config(&config, attributes, stream);
    const long long tiles = (long long)((M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + 255) / 256);
    config.gridDim = dim3(2u * (unsigned)(tiles < slots ? tiles : slots));
    config.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t status = cudaLaunchKernelEx(&config, gemm_tcgen05_pair_kernel<PAIR_STAGES>, map_a, map_w, map_out,
                                                  tma_out, out, M, N, K, mode, act, flag, rope);
    if (status != cudaSuccess) return fail("skv_linear(tcgen05 pair)", cudaGetErrorString(status));
    return 0;
}

// Whether the two-block kernel is the cheaper one, in the units of the cost of a width below (rounds x 256 columns):
// measured against 256-wide tiles of one block it is 4-6 % faster where the main loop dominates (2,048 x 11,264 x 2,048:
// 71.3 -> 67.7 us; 2,048 x 2,048 x 5,632: 36.5 -> 34.9; 8,192 cubed: 806 -> 768, the library GEMM 779-816) and 4 %
// slower where a block has one short tile (2,048 x 2,048 x 2,048: 16.0 -> 16.6 us; a pair's set-up is heavier).
static double pair_cost(int M, int N, int K) {
    const int slots = pair_slots();
    if (slots <= 0 || N <= 128) return 1e30;
    const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    const long long rounds = (tiles + slots - 1) / slots;
    if (rounds * ((K + TC_BK - 1) / TC_BK) < 80) return 1e30;
    return (double)rounds * 256 / 1.04;
}

template <int MP, int STAGES, int CH>
static int launch_few_tokens(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                             int* flag, cudaStream_t stream) {
    CUtensorMap map_w, map_x;
    if (CH == 1) {
        if (int code = tensor_map(w, N, K, 2, 128, TC_BK, &map_w)) return code;
        if (int code = tensor_map(a, M, K, 2, MP, TC_BK, &map_x)) return code;
    } else {
        if (K % TC_BK != 0) return fail("skv_linear(tcgen05)", "copies of several chunks need an inner size that is a multiple of 64");
        if (int code = tensor_map_chunks(w, N, K, 128, CH, &map_w)) return code;
        if (int code = tensor_map_chunks(a, M, K, MP, CH, &map_x)) return code;
    }
    constexpr size_t ring = (size_t)STAGES * CH * (128 * TC_BK * 2 + MP * TC_BK * 2);
    constexpr size_t smem = ring + (2 * STAGES + 1) * 8 + 16 + 1024;
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            return fail("skv_linear(tcgen05)", "cannot read the number of SMs");
        cudaError_t status = cudaFuncSetAttribute(gemm_tcgen05_few_tokens_kernel<MP, STAGES, CH>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_linear(tcgen05)", cudaGetErrorString(status));
        sm_count = count;
    }
    // Parts of K per tile of 128 weight rows: the largest power of two up to 4 (eight ranks pushing into one block
    // measured slower than four) that keeps the grid within the GPU, leaves
    // every part at least four 64-wide steps, and whose partial results fit where the pipeline's stages were.
    const int n_tiles = (N + 127) / 128, k_blocks = (K + TC_BK - 1) / TC_BK;
    int splits = 1;
    while (splits < 4 && n_tiles * splits * 2 <= sm_count && k_blocks >= splits * 2 * 4 &&
           (size_t)(splits * 2 - 1) * MP * 128 * 4 <= ring)
        splits *= 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)n_tiles, (unsigned)splits, 1);
    config.blockDim = dim3(TC_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = (unsigned)splits;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t status = cudaLaunchKernelEx(&config, gemm_tcgen05_few_tokens_kernel<MP, STAGES, CH>, map_w, map_x, out,
                                                  M, N, K, mode, act, splits, flag);
    if (status != cudaSuccess) return fail("skv_linear(tcgen05)", cudaGetErrorString(status));
    return 0;
}

// Which kernel serves a shape.  Up to 128 tokens the few-token kernel.  Above, a tile form by cost: wider tiles re-read
// less of A and W from L2 per flop (measured at 2,048 x 6,144 x 4,096: 1,268 TFLOP/s with 256-wide tiles, 1,014 with
// 160, 860 with 128); narrow ones waste less on small N and fill the last round of tiles better: 2,048 tokens x
// 2,560 columns are 160 tiles of 256 columns (two rounds on 148 SMs, the second nearly empty: 27.9 us) but 256 tiles of
// 160 (two rounds of five eighths the work: 25.6 us).  Cost of a width: rounds x width / efficiency per flop.  A width
// of 160 serves the float epilogues only (its slabs of 32 columns divide it; the 64- and 128-column slabs of the
// other modes do not).
enum { FORM_FEW_TOKENS = 0, FORM_128 = 1, FORM_160 = 2, FORM_256 = 3, FORM_PAIR = 4 };

// (Tried: a width of 192 for the bfloat16 store and, at head size 64, the rotary epilogue.  The q|k|v projection of
// 2,048 tokens x 2,560 columns, 224 tiles of 192 instead of 160 of 256, took 29.5 us against 27.8 with the rotary
// epilogue, whose work per tile does not shrink with the width; the prefill did not move.)
static int choose_form(int M, int N, int K, int mode) {
    if (M <= 128) return FORM_FEW_TOKENS;
    const long long m_tiles = (M + 127) / 128;
    auto cost = [&](int width, double efficiency) {
        const long long tiles = m_tiles * ((N + width - 1) / width);
        return (double)((tiles + tc_sm_count() - 1) / tc_sm_count()) * width / efficiency;
    };
    const bool float_out = mode == TC_MODE_STORE_F32 || mode == TC_MODE_ADD_F32;
    const double wide = N > 128 ? cost(256, 1.0) : 1e30, narrow = cost(128, 0.68);
    const double middle = (float_out && N > 128) ? cost(160, 0.80) : 1e30;
    const double paired = pair_cost(M, N, K);
    if (paired < wide && paired < middle && paired < narrow) return FORM_PAIR;
    if (middle < wide && middle < narrow) return FORM_160;
    return wide <= narrow ? FORM_256 : FORM_128;
}

int linear_tcgen05(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act, int* flag,
                   cudaStream_t stream) {
    if (K % 8 != 0) return fail("skv_linear(tcgen05)", "the inner size must be a multiple of 8 (16-byte rows)");
    if (((uintptr_t)a | (uintptr_t)w) & 15) return fail("skv_linear(tcgen05)", "operands must be 16-byte aligned");
    if (mode == TC_MODE_GATED && N % 16 != 0) return fail("skv_linear(tcgen05)", "a gated weight needs a multiple of 16 rows");
    // More tiles of 128 weight rows than SMs: rings half as deep, so that two blocks share an SM and one's set-up and
    // epilogue run under the other's stream (64 tokens, 22,016 x 4,096: 54.0 -> 39.3 us; 28,672 x 4,096: 56.0 -> 46.0;
    // 32,000 x 2,048: 26.3 -> 23.4).  With fewer tiles the deep ring of a block alone on its SM is faster (2,048 x
    // 5,632: 10.0 against 12.6 us).
    const bool many_tiles = (N + 127) / 128 > tc_sm_count();
    // (copies of two chunks where K allows it and the blocks are few enough for each to be limited by what it can keep
    // on its way; see the kernel)
    const bool two_chunks = K % TC_BK == 0 && !many_tiles;
    if (M <= 32) return many_tiles ? launch_few_tokens<32, 4, 1>(a, w, out, M, N, K, mode, act, flag, stream)
                       : two_chunks ? launch_few_tokens<32, 4, 2>(a, w, out, M, N, K, mode, act, flag, stream)
                                    : launch_few_tokens<32, 8, 1>(a, w, out, M, N, K, mode, act, flag, stream);
    if (M <= 64) return many_tiles ? launch_few_tokens<64, 4, 1>(a, w, out, M, N, K, mode, act, flag, stream)
                       : two_chunks ? launch_few_tokens<64, 4, 2>(a, w, out, M, N, K, mode, act, flag, stream)
                                    : launch_few_tokens<64, 8, 1>(a, w, out, M, N, K, mode, act, flag, stream);
    if (M <= 128) return many_tiles ? launch_few_tokens<128, 3, 1>(a, w, out, M, N, K, mode, act, flag, stream)
                        : two_chunks ? launch_few_tokens<128, 3, 2>(a, w, out, M, N, K, mode, act, flag, stream)
                                     : launch_few_tokens<128, 6, 1>(a, w, out, M, N, K, mode, act, flag, stream);
    switch (choose_form(M, N, K, mode)) {
        case FORM_PAIR: return launch_pair(a, w, out, M, N, K, mode, act, flag, stream);
        case FORM_160: return launch_tc<160, 5>(a, w, out, M, N, K, mode, act, flag, stream);
        case FORM_256: return launch_tc<256, 4>(a, w, out, M, N, K, mode, act, flag, stream);
        default: return launch_tc<128, 4>(a, w, out, M, N, K, mode, act, flag, stream);
    }
}

// The q|k|v projection of a step with many tokens, with the rotary encoding and the cache write in its epilogue.
int linear_tcgen05_qkv_rope(const void* a, const void* w, void* q_out, int M, int N, int K, const RopeArgs& rope,
                            int* flag, cudaStream_t stream) {
    if (K % 8 != 0) return fail("skv_linear_qkv_rope", "the inner size must be a multiple of 8 (16-byte rows)");
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)q_out | (uintptr_t)rope.k_cache | (uintptr_t)rope.v_cache |
         (uintptr_t)rope.cos_sin) & 15)
        return fail("skv_linear_qkv_rope", "operands must be 16-byte aligned");
    if (M <= 128) return fail("skv_linear_qkv_rope", "this form serves steps of more than 128 tokens");
    if (rope.head_dim != 64 && rope.head_dim != 128) return fail("skv_linear_qkv_rope", "head size 64 or 128 only");
    if (rope.num_heads <= 0 || rope.num_kv_heads <= 0 || N != (rope.num_heads + 2 * rope.num_kv_heads) * rope.head_dim)
        return fail("skv_linear_qkv_rope", "the weight's rows must be [query heads | key heads | value heads]");
    if (rope.block_size <= 0 || rope.table_width <= 0) return fail("skv_linear_qkv_rope", "bad cache block size or table width");
    switch (choose_form(M, N, K, TC_MODE_QKV_ROPE)) {
        case FORM_PAIR: return launch_pair(a, w, q_out, M, N, K, TC_MODE_QKV_ROPE, 0, flag, stream, rope);
        case FORM_256: return launch_tc<256, 4>(a, w, q_out, M, N, K, TC_MODE_QKV_ROPE, 0, flag, stream, rope);
        default: return launch_tc<128, 4>(a, w, q_out, M, N, K, TC_MODE_QKV_ROPE, 0, flag, stream, rope);
    }
}

}  // namespace skv

using namespace skv;

SKV_EXPORT int skv_has_linear_qkv_rope() { return 1; }

// Which of the tensor-memory kernels serves a projection of this shape and epilogue on this GPU (0 the few-token
// kernel, 1-3 tiles of 128, 160 and 256 columns, 4 the two-block kernel): for tests, which have to know that the
// shapes they bring reach every one of them.
SKV_EXPORT int skv_linear_tcgen05_form(int M, int N, int K, int mode) { return choose_form(M, N, K, mode); }

// out q [M, heads x head_dim] bfloat16 = rotated (a[M, K] . w[N, K]^T)[:, query columns]; keys (rotated) and values
// of token m go to the cache row of position positions[m] of sequence token_seq[m] if write_kv.  See RopeArgs.
SKV_EXPORT int skv_linear_qkv_rope(const void* a, const void* w, void* q_out, int M, int N, int K, const float* cos_sin,
                                   const int* positions, const int* token_seq, const int* block_table, int table_width,
                                   void* k_cache, void* v_cache, int num_heads, int num_kv_heads, int head_dim,
                                   int block_size, int write_kv, int* flag, cudaStream_t stream) {
    if (M <= 0) return 0;
    RopeArgs rope;
    rope.cos_sin = (const float2*)cos_sin;
    rope.positions = positions;
    rope.token_seq = token_seq;
    rope.block_table = block_table;
    rope.k_cache = (__nv_bfloat16*)k_cache;
    rope.v_cache = (__nv_bfloat16*)v_cache;
    rope.table_width = table_width;
    rope.num_heads = num_heads;
    rope.num_kv_heads = num_kv_heads;
    rope.head_dim = head_dim;
    rope.block_size = block_size;
    rope.write_kv = write_kv;
    return linear_tcgen05_qkv_rope(a, w, q_out, M, N, K, rope, flag, stream);
}

#else

SKV_EXPORT int skv_has_linear_qkv_rope() { return 0; }

SKV_EXPORT int skv_linear_tcgen05_form(int, int, int, int) { return -1; }

SKV_EXPORT int skv_linear_qkv_rope(const void*, const void*, void*, int, int, int, const float*, const int*, const int*,
                                   const int*, int, void*, void*, int, int, int, int, int, int*, cudaStream_t) {
    return skv::fail("skv_linear_qkv_rope", "only the bfloat16 build has this kernel");
}

#endif
