// Prefill attention for bfloat16: many new tokens per sequence, causal, grouped-query,
// reading keys and values from the paged cache (so a prompt may continue one that is
// already cached).
//
// The reference has no prefill kernel: its GPU path feeds a prompt one token at a time
// through paged_attention_decode_kernel (src/generation/generator.cpp:661-688).  This is
// the flash-attention form of the same arithmetic (src/layers/attention.cpp:261-338):
// a block takes 64 queries of one head of one sequence, its 4 warps 16 queries each;
// keys and values stream through shared memory in tiles of 64 (cp.async, two buffers);
// scores and the output accumulate in float in mma.sync m16n8k16 fragments with an
// online softmax; the scale multiplies the finished dot product; a query at absolute
// position p sees keys lo..p (lo = 0 or p - window + 1).
#include "common.cuh"

#if SKV_DTYPE == SKV_BF16 && SKV_HEAD_DIM <= 128

namespace skv {

constexpr int PHD = SKV_HEAD_DIM;
constexpr int PF_BM = 64, PF_BN = 64, PF_WARPS = 4;
constexpr int PF_PITCH = PHD + 8;                 // elements; 16 bytes of padding per row
constexpr int PF_KSTEPS = PHD / 16, PF_DTILES = PHD / 8;

__device__ __forceinline__ void pf_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool live) {
    const int bytes = live ? 16 : 0;              // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// 2^x by the special-function unit.  Scores are kept multiplied by log2(e), so that
// exp(s - m) = 2^(s' - m'); the unit's error (about 2 ulp of float) is far below the
// bfloat16 rounding the probabilities get before they multiply V.
__device__ __forceinline__ float pf_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}

__global__ void __launch_bounds__(PF_WARPS * 32)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_after,
                         __nv_bfloat16* __restrict__ out, int num_heads, int num_kv_heads, int block_size,
                         float scale, int window, int tiles_per_seq) {
    extern __shared__ __align__(16) uint8_t pf_smem[];      // [2 buffers][K tile | V tile]
    constexpr int TILE_ELEMS = PF_BN * PF_PITCH;
    __nv_bfloat16* tiles = (__nv_bfloat16*)pf_smem;
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x / tiles_per_seq, tile = blockIdx.x - seq * tiles_per_seq;
    const int head = blockIdx.y;
    const int kv_head = head / (num_heads / num_kv_heads);
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    if (tile * PF_BM >= q_len) return;                       // the whole block leaves together
    const int ctx = ctx_after[seq], ctx_before = ctx - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int row0 = tile * PF_BM + warp * 16;               // this warp's first query (index among the new tokens)
    const int* table = block_table + (size_t)seq * table_width;

    // key range of the block: every key a query of this tile may see
    const int last_query = min(q_len, tile * PF_BM + PF_BM) - 1;
    const int kv_end = ctx_before + last_query + 1;          // exclusive
    const int kv_lo = window > 0 ? max(0, ctx_before + tile * PF_BM - window + 1) : 0;
    const int first_tile = kv_lo / PF_BN, end_tile = (kv_end + PF_BN - 1) / PF_BN;

    // Q fragments straight from global memory (rows g and g+8 of the warp's 16)
    uint32_t qa[PF_KSTEPS][4];
    {
        const int r_top = row0 + g, r_bottom = row0 + g + 8;
        const __nv_bfloat16* top = q + ((size_t)(q_begin + min(r_top, q_len - 1)) * num_heads + head) * PHD;
        const __nv_bfloat16* bottom = q + ((size_t)(q_begin + min(r_bottom, q_len - 1)) * num_heads + head) * PHD;
#pragma unroll
        for (int s = 0; s < PF_KSTEPS; ++s) {
            qa[s][0] = r_top < q_len ? *(const uint32_t*)(top + 16 * s + 2 * tig) : 0u;
            qa[s][1] = r_bottom < q_len ? *(const uint32_t*)(bottom + 16 * s + 2 * tig) : 0u;
            qa[s][2] = r_top < q_len ? *(const uint32_t*)(top + 16 * s + 8 + 2 * tig) : 0u;
            qa[s][3] = r_bottom < q_len ? *(const uint32_t*)(bottom + 16 * s + 8 + 2 * tig) : 0u;
        }
    }
    const int pos_top = ctx_before + row0 + g, pos_bottom = pos_top + 8;   // absolute positions of the two rows
    const float scale_log2 = scale * 1.4426950408889634f;                  // scores in units of log2

    auto load_tile = [&](int kt, int buffer) {
        __nv_bfloat16* k_dst = tiles + (size_t)buffer * 2 * TILE_ELEMS;
        __nv_bfloat16* v_dst = k_dst + TILE_ELEMS;
        constexpr int CHUNKS = PHD / 8;                      // 16-byte chunks per row
        for (int idx = threadIdx.x; idx < PF_BN * CHUNKS; idx += PF_WARPS * 32) {
            const int r = idx / CHUNKS, c = idx - r * CHUNKS;
            const int key = kt * PF_BN + r;
            const bool live = key < ctx;
            const int safe = live ? key : 0;
            const int block = table[safe / block_size];
            const size_t at = ((size_t)(block * num_kv_heads + kv_head) * block_size + (safe % block_size)) * PHD + c * 8;
            cp_async_16(smem_u32(k_dst + r * PF_PITCH + c * 8), k_cache + at, live);
            cp_async_16(smem_u32(v_dst + r * PF_PITCH + c * 8), v_cache + at, live);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float o[PF_DTILES][4];
#pragma unroll
    for (int j = 0; j < PF_DTILES; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};

    if (first_tile < end_tile) load_tile(first_tile, 0);
    for (int kt = first_tile; kt < end_tile; ++kt) {
        const int buffer = (kt - first_tile) & 1;
        if (kt + 1 < end_tile) {
            load_tile(kt + 1, buffer ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* k_tile = tiles + (size_t)buffer * 2 * TILE_ELEMS;
        const __nv_bfloat16* v_tile = k_tile + TILE_ELEMS;
        // this warp needs the tile only if one of its queries can see one of its keys
        const int warp_last_pos = ctx_before + min(row0 + 15, q_len - 1);
        const bool warp_active = row0 < q_len && kt * PF_BN <= warp_last_pos;
        if (warp_active) {
            float s[PF_BN / 8][4];
#pragma unroll
            for (int n = 0; n < PF_BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f; }
#pragma unroll
            for (int step = 0; step < PF_KSTEPS; ++step) {
#pragma unroll
                for (int n2 = 0; n2 < PF_BN / 16; ++n2) {
                    // four 8x8 matrices: (keys 16n2..+7, d 16step..+7), (same keys, d +8), (keys +8, d), (keys +8, d +8)
                    const int id = lane >> 3, r = lane & 7;
                    const __nv_bfloat16* src = k_tile + (16 * n2 + (id >> 1) * 8 + r) * PF_PITCH + 16 * step + (id & 1) * 8;
                    uint32_t kb[4];
                    ldmatrix_x4(kb, smem_u32(src));
                    pf_mma(s[2 * n2], qa[step][0], qa[step][1], qa[step][2], qa[step][3], kb[0], kb[1]);
                    pf_mma(s[2 * n2 + 1], qa[step][0], qa[step][1], qa[step][2], qa[step][3], kb[2], kb[3]);
                }
            }
            // scale and mask
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < PF_BN / 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kt * PF_BN + 8 * n + 2 * tig + (c & 1);
                    const int pos = (c >> 1) ? pos_bottom : pos_top;
                    const bool seen = key <= pos && (window == 0 || key > pos - window);
                    const float v = seen ? s[n][c] * scale_log2 : -INFINITY;
                    s[n][c] = v;
                    tile_max[c >> 1] = fmaxf(tile_max[c >> 1], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m = tile_max[r];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                const float new_max = fmaxf(row_max[r], m);
                corr[r] = new_max == -INFINITY ? 1.0f : pf_exp2(row_max[r] - new_max);
                row_max[r] = new_max;
            }
            float partial[2] = {0.0f, 0.0f};
#pragma unroll
            for (int n = 0; n < PF_BN / 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float m = row_max[c >> 1];
                    const float p = m == -INFINITY ? 0.0f : pf_exp2(s[n][c] - m);
                    s[n][c] = p;
                    partial[c >> 1] += p;
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * corr[r] + partial[r];
#pragma unroll
            for (int j = 0; j < PF_DTILES; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
#pragma unroll
            for (int ks = 0; ks < PF_BN / 16; ++ks) {
                const uint32_t a0 = pf_pack(s[2 * ks][0], s[2 * ks][1]), a1 = pf_pack(s[2 * ks][2], s[2 * ks][3]);
                const uint32_t a2 = pf_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pf_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                for (int d2 = 0; d2 < PF_DTILES / 2; ++d2) {
                    // transposed 8x8 matrices: (keys 16ks..+7, d 16d2..+7), (keys +8, same d), (keys, d +8), (keys +8, d +8)
                    const int id = lane >> 3, r = lane & 7;
                    const __nv_bfloat16* src = v_tile + (16 * ks + (id & 1) * 8 + r) * PF_PITCH + 16 * d2 + (id >> 1) * 8;
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, smem_u32(src));
                    pf_mma(o[2 * d2], a0, a1, a2, a3, vb[0], vb[1]);
                    pf_mma(o[2 * d2 + 1], a0, a1, a2, a3, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();                                      // the buffer may be refilled now
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    const int r_top = row0 + g, r_bottom = row0 + g + 8;
    const float inv_top = 1.0f / row_sum[0], inv_bottom = 1.0f / row_sum[1];
#pragma unroll
    for (int j = 0; j < PF_DTILES; ++j) {
        const int d = 8 * j + 2 * tig;
        if (r_top < q_len)
            *(uint32_t*)(out + ((size_t)(q_begin + r_top) * num_heads + head) * PHD + d) =
                pf_pack(o[j][0] * inv_top, o[j][1] * inv_top);
        if (r_bottom < q_len)
            *(uint32_t*)(out + ((size_t)(q_begin + r_bottom) * num_heads + head) * PHD + d) =
                pf_pack(o[j][2] * inv_bottom, o[j][3] * inv_bottom);
    }
}

}  // namespace skv

using namespace skv;

// Sequences' new tokens are packed: sequence s owns rows cu_q[s] .. cu_q[s+1]-1 of q and out, and
// ctx_after[s] keys are cached for it after this step's keys were written.
SKV_EXPORT int skv_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                                     const int* block_table, int table_width, const int* cu_q,
                                     const int* ctx_after, void* out, int n_seqs, int max_q_len, int num_heads,
                                     int num_kv_heads, int head_dim, int block_size, float scale, int window,
                                     cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (head_dim != PHD) return fail("skv_attention_prefill", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_prefill", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || window < 0) return fail("skv_attention_prefill", "bad block size or window");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)
        return fail("skv_attention_prefill", "operands must be 16-byte aligned");
    const int tiles_per_seq = (max_q_len + PF_BM - 1) / PF_BM;
    const long long blocks = (long long)n_seqs * tiles_per_seq;
    if (blocks > 0x7fffffffLL || num_heads > 65535) return fail("skv_attention_prefill", "too many tokens or heads");
    const size_t smem = (size_t)2 * 2 * PF_BN * PF_PITCH * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(prefill_attention_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_attention_prefill", cudaGetErrorString(status));
        configured = true;
    }
    return launch_pdl("skv_attention_prefill", prefill_attention_kernel, dim3((unsigned)blocks, num_heads),
                      dim3(PF_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                      (const __nv_bfloat16*)v_cache, block_table, table_width, cu_q, ctx_after, (__nv_bfloat16*)out,
                      num_heads, num_kv_heads, block_size, scale, window, tiles_per_seq);
}

SKV_EXPORT int skv_has_attention_prefill() { return 1; }

#else

SKV_EXPORT int skv_attention_prefill(const void*, const void*, const void*, const int*, int, const int*, const int*,
                                     void*, int, int, int, int, int, int, float, int, cudaStream_t) {
    return skv::fail("skv_attention_prefill", "this build (float32, or a head size above 128) uses skv_attention");
}

SKV_EXPORT int skv_has_attention_prefill() { return 0; }

#endif
