// Decode attention with its neighbours folded in (bfloat16): rotary encoding of the new
// token's queries and key, the write of that key and value into the paged cache, the
// split-KV attention itself, and the merge of the splits, as one kernel.
//
// It replaces four launches of the unfused path (rope_kv_write_kernel, decode_attention_kernel,
// decode_combine_kernel; in the reference: generate_rope_frequencies, rope_split_half x2, two
// cache-append copies and paged_attention_decode_kernel, src/models/transformer_block.cpp:
// 457-518).  The arithmetic is the same as in elementwise.cu and attention_decode.cu: pairs
// (i, i + head_dim/2) rotate in float with a host-built cos/sin table, queries and keys are
// rounded to bfloat16 once, scores / softmax / output accumulate in float.
//
// The splits of one (sequence, KV head) are the blocks of a thread-block cluster: each block
// leaves its partial (max, sum, output) in its own shared memory and, after a cluster barrier,
// the blocks share out the rows and read one another's partials through distributed shared
// memory.  No scratch in global memory, no second kernel.  The block whose split holds the
// newest position writes that token's key and value to the cache before it reads them.
#include "common.cuh"

#if SKV_DTYPE == SKV_BF16

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace skv {

constexpr int FHD = SKV_HEAD_DIM;
constexpr int FKSTEPS = FHD / 16, FOTILES = FHD / 8, FVWORDS = FHD / 16;
constexpr int FWARPS = 8;
constexpr int FPITCH = FHD + 2;

__device__ __forceinline__ void f_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float f_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t f_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}

// element d of a head after rotation; x points at the head's head_dim floats, angles at the
// position's head_dim/2 (cos, sin) pairs (null: no rotation)
__device__ __forceinline__ float rotated(const float* x, const float2* angles, int d) {
    constexpr int HALF = FHD / 2;
    if (!angles) return x[d];
    if (d < HALF) { const float2 a = angles[d]; return x[d] * a.x - x[d + HALF] * a.y; }
    const float2 a = angles[d - HALF];
    return x[d - HALF] * a.y + x[d] * a.x;
}

__global__ void __launch_bounds__(FWARPS * 32, FHD <= 64 ? 2 : 1)
decode_attention_fused_kernel(const float* __restrict__ qkv, const float2* __restrict__ cos_sin,
                              __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                              const int* __restrict__ block_table, int table_width,
                              const int* __restrict__ ctx_after, __nv_bfloat16* __restrict__ out, int num_heads,
                              int num_kv_heads, int block_size, float scale, int window, int splits, int m_tiles,
                              int write_kv) {
    extern __shared__ float fused_smem[];             // [warps][16][FPITCH] merge area, then [16][FPITCH] result
    float* result = fused_smem + (size_t)FWARPS * 16 * FPITCH;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int seq = blockIdx.x;
    const int kv_head = blockIdx.y / m_tiles, m_tile = blockIdx.y - kv_head * m_tiles;
    const int split = blockIdx.z;
    const int group_size = num_heads / num_kv_heads;
    const int head0 = kv_head * group_size + m_tile * 16;
    const int rows = min(16, group_size - m_tile * 16);
    const int q_dim = num_heads * FHD, kv_dim = num_kv_heads * FHD;

    const int ctx = ctx_after[seq];
    const int pos = ctx - 1;                          // the new token's position
    const int lo = window > 0 ? max(0, ctx - window) : 0;
    const int first_group = lo >> 4, end_group = (ctx + 15) >> 4;
    const int per_split = (end_group - first_group + splits - 1) / splits;
    const int my_first = first_group + split * per_split;
    const int my_end = min(end_group, my_first + per_split);
    const int* table = block_table + (size_t)seq * table_width;
    const float scale_log2 = scale * 1.4426950408889634f;
    const float* token = qkv + (size_t)seq * (q_dim + 2 * kv_dim);
    const float2* angles = cos_sin ? cos_sin + (size_t)pos * (FHD / 2) : nullptr;

    // One group of 16 keys: the lane's share of its keys (for Q.K^T) and values (for P.V), in registers.
    struct GroupData { uint2 kb[2][FKSTEPS]; uint32_t vw[4][FVWORDS]; };
    auto load_group = [&](int group, GroupData& data) {
        const int j0 = group << 4;
        const int block = table[j0 / block_size];
        const size_t base = ((size_t)(block * num_kv_heads + kv_head) * block_size + (j0 % block_size)) * FHD;
        const __nv_bfloat16* k_rows = k_cache + base;
        const __nv_bfloat16* v_rows = v_cache + base;
        const int keys[4] = {2 * tig, 2 * tig + 1, 2 * tig + 8, 2 * tig + 9};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool live = j0 + keys[i] < ctx;
            const uint32_t* src = (const uint32_t*)(v_rows + (size_t)keys[i] * FHD + g * (FHD / 8));
#pragma unroll
            for (int w = 0; w < FVWORDS; ++w) data.vw[i][w] = live ? src[w] : 0u;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const bool live = j0 + 8 * t + g < ctx;
            const __nv_bfloat16* key_row = k_rows + (size_t)(8 * t + g) * FHD + 4 * tig;
#pragma unroll
            for (int step = 0; step < FKSTEPS; ++step)
                data.kb[t][step] = live ? *(const uint2*)(key_row + 16 * step) : make_uint2(0u, 0u);
        }
    };
    // Keys and values of earlier positions were written by earlier steps, so the warp's first group can be
    // fetched before waiting for the kernel in front (the q|k|v projection): the loads overlap its end.  Not
    // the group that holds the new position, and not for a layer that reads a cache another layer of this
    // same step writes (write_kv == 0).
    const int newest_group = pos >> 4;
    const int first_mine = my_first + warp;
    const bool prefetched = write_kv && first_mine < my_end && first_mine != newest_group;
    GroupData ahead;
    if (prefetched) load_group(first_mine, ahead);
    pdl_wait();

    // the block whose split holds the newest position puts that token's key and value in the cache
    if (write_kv && newest_group >= my_first && newest_group < my_end) {
        const int block = table[pos / block_size];
        const size_t at = ((size_t)(block * num_kv_heads + kv_head) * block_size + (pos % block_size)) * FHD;
        const float* k_new = token + q_dim + (size_t)kv_head * FHD;
        const float* v_new = token + q_dim + kv_dim + (size_t)kv_head * FHD;
        for (int d = threadIdx.x; d < FHD; d += blockDim.x) {
            k_cache[at + d] = __float2bfloat16_rn(rotated(k_new, angles, d));
            v_cache[at + d] = __float2bfloat16_rn(v_new[d]);
        }
        __threadfence_block();
    }
    __syncthreads();                                  // the block's later loads of that row see the stores

    // rotated query fragments: rows g and g+8 are heads head0+g, head0+g+8; elements 16s + 4tig .. +3
    uint32_t qa[FKSTEPS][4];
#pragma unroll
    for (int s = 0; s < FKSTEPS; ++s) {
        float top[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bottom[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (g < rows) {
            const float* x = token + (size_t)(head0 + g) * FHD;
#pragma unroll
            for (int e = 0; e < 4; ++e) top[e] = rotated(x, angles, 16 * s + 4 * tig + e);
        }
        if (g + 8 < rows) {
            const float* x = token + (size_t)(head0 + g + 8) * FHD;
#pragma unroll
            for (int e = 0; e < 4; ++e) bottom[e] = rotated(x, angles, 16 * s + 4 * tig + e);
        }
        qa[s][0] = f_pack(top[0], top[1]); qa[s][1] = f_pack(bottom[0], bottom[1]);
        qa[s][2] = f_pack(top[2], top[3]); qa[s][3] = f_pack(bottom[2], bottom[3]);
    }

    float o[FOTILES][4];
#pragma unroll
    for (int j = 0; j < FOTILES; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};

    for (int group = first_mine; group < my_end; group += FWARPS) {
        const int j0 = group << 4;
        GroupData data;
        if (group == first_mine && prefetched) data = ahead;
        else load_group(group, data);
        float s[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.0f;
#pragma unroll
            for (int step = 0; step < FKSTEPS; ++step)
                f_mma(s[t], qa[step][0], qa[step][1], qa[step][2], qa[step][3], data.kb[t][step].x, data.kb[t][step].y);
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int t = 0; t < 2; ++t) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = j0 + 8 * t + 2 * tig + (c & 1);
                const float v = (key < ctx && key >= lo) ? s[t][c] * scale_log2 : -INFINITY;
                s[t][c] = v;
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
            corr[r] = new_max == -INFINITY ? 1.0f : f_exp2(row_max[r] - new_max);
            row_max[r] = new_max;
        }
        float p[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float m = row_max[c >> 1];
                p[t][c] = m == -INFINITY ? 0.0f : f_exp2(s[t][c] - m);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
            row_sum[r] = row_sum[r] * corr[r] + p[0][2 * r] + p[0][2 * r + 1] + p[1][2 * r] + p[1][2 * r + 1];
#pragma unroll
        for (int j = 0; j < FOTILES; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        const uint32_t a0 = f_pack(p[0][0], p[0][1]), a1 = f_pack(p[0][2], p[0][3]);
        const uint32_t a2 = f_pack(p[1][0], p[1][1]), a3 = f_pack(p[1][2], p[1][3]);
#pragma unroll
        for (int w = 0; w < FVWORDS; ++w) {
            f_mma(o[2 * w], a0, a1, a2, a3, __byte_perm(data.vw[0][w], data.vw[1][w], 0x5410),
                  __byte_perm(data.vw[2][w], data.vw[3][w], 0x5410));
            f_mma(o[2 * w + 1], a0, a1, a2, a3, __byte_perm(data.vw[0][w], data.vw[1][w], 0x7632),
                  __byte_perm(data.vw[2][w], data.vw[3][w], 0x7632));
        }
    }
    // merge the warps into `result`: rows x (head_dim outputs, max, sum)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    float* mine = fused_smem + (size_t)warp * 16 * FPITCH;
#pragma unroll
    for (int j = 0; j < FOTILES; ++j) {
        const int d0 = (2 * tig) * (FHD / 8) + j, d1 = (2 * tig + 1) * (FHD / 8) + j;
        mine[g * FPITCH + d0] = o[j][0];
        mine[g * FPITCH + d1] = o[j][1];
        mine[(g + 8) * FPITCH + d0] = o[j][2];
        mine[(g + 8) * FPITCH + d1] = o[j][3];
    }
    if (tig == 0) {
        mine[g * FPITCH + FHD] = row_max[0];
        mine[g * FPITCH + FHD + 1] = row_sum[0];
        mine[(g + 8) * FPITCH + FHD] = row_max[1];
        mine[(g + 8) * FPITCH + FHD + 1] = row_sum[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * FPITCH; idx += blockDim.x) {
        const int r = idx / FPITCH, d = idx - r * FPITCH;
        float m = -INFINITY;
        for (int w = 0; w < FWARPS; ++w) m = fmaxf(m, fused_smem[((size_t)w * 16 + r) * FPITCH + FHD]);
        float value;
        if (d == FHD) {
            value = m;
        } else {
            float total = 0.0f;
            if (m != -INFINITY) {
                for (int w = 0; w < FWARPS; ++w) {
                    const float* tile = fused_smem + ((size_t)w * 16 + r) * FPITCH;
                    total += f_exp2(tile[FHD] - m) * tile[d];      // column FHD+1 (the sums) is weighted the same way
                }
            }
            value = total;
        }
        result[idx] = value;
    }
    if (splits == 1) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < rows * FHD; idx += blockDim.x) {
            const int r = idx / FHD, d = idx - r * FHD;
            out[((size_t)seq * num_heads + head0 + r) * FHD + d] =
                __float2bfloat16_rn(result[r * FPITCH + d] / result[r * FPITCH + FHD + 1]);
        }
        return;
    }
    // merge the splits: the cluster's blocks share out the rows and read every block's `result`
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int rank = (int)cluster.block_rank(), blocks = (int)cluster.num_blocks();
    for (int idx = threadIdx.x; idx < rows * FHD; idx += blockDim.x) {
        const int r = idx / FHD, d = idx - r * FHD;
        if (r % blocks != rank) continue;
        float m = -INFINITY;
        for (int b = 0; b < blocks; ++b) m = fmaxf(m, cluster.map_shared_rank(result, b)[r * FPITCH + FHD]);
        float total = 0.0f, sum = 0.0f;
        for (int b = 0; b < blocks; ++b) {
            const float* remote = cluster.map_shared_rank(result, b);
            const float mb = remote[r * FPITCH + FHD];
            if (mb == -INFINITY) continue;
            const float weight = f_exp2(mb - m);
            total += weight * remote[r * FPITCH + d];
            sum += weight * remote[r * FPITCH + FHD + 1];
        }
        out[((size_t)seq * num_heads + head0 + r) * FHD + d] = __float2bfloat16_rn(total / sum);
    }
    cluster.sync();                                   // nobody leaves while its shared memory is being read
}

}  // namespace skv

using namespace skv;

// qkv: float [n_seqs, (heads + 2 kv_heads) * head_dim] (the q|k|v projection of each sequence's new
// token); cos_sin: float [positions, head_dim/2, 2] or null; ctx_after[s]: keys cached for sequence s
// once this token's key is in (so the token's position is ctx_after[s] - 1).  splits is 1..8.
SKV_EXPORT int skv_attention_decode_fused(const float* qkv, const float* cos_sin, void* k_cache, void* v_cache,
                                          const int* block_table, int table_width, const int* ctx_after,
                                          void* out, int n_seqs, int num_heads, int num_kv_heads, int head_dim,
                                          int block_size, float scale, int window, int splits, int write_kv,
                                          cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (head_dim != FHD) return fail("skv_attention_decode_fused", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_decode_fused", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || block_size % 16 != 0)
        return fail("skv_attention_decode_fused", "block_size must be a positive multiple of 16");
    if (splits < 1 || splits > 8) return fail("skv_attention_decode_fused", "splits must be 1..8 (one cluster)");
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)qkv) & 15)
        return fail("skv_attention_decode_fused", "operands must be 16-byte aligned");
    const int group_size = num_heads / num_kv_heads;
    const int m_tiles = (group_size + 15) / 16;
    const size_t smem = (size_t)(FWARPS + 1) * 16 * FPITCH * sizeof(float);
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(decode_attention_fused_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_attention_decode_fused", cudaGetErrorString(status));
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(n_seqs, num_kv_heads * m_tiles, splits);
    config.blockDim = dim3(FWARPS * 32);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = splits;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t status = cudaLaunchKernelEx(
        &config, decode_attention_fused_kernel, qkv, (const float2*)cos_sin, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, block_table, table_width, ctx_after, (__nv_bfloat16*)out, num_heads, num_kv_heads,
        block_size, scale, window, splits, m_tiles, write_kv);
    if (status != cudaSuccess) return fail("skv_attention_decode_fused", cudaGetErrorString(status));
    return 0;
}

#else

SKV_EXPORT int skv_attention_decode_fused(const float*, const float*, void*, void*, const int*, int, const int*, void*,
                                          int, int, int, int, int, float, int, int, int, cudaStream_t) {
    return skv::fail("skv_attention_decode_fused", "only the bfloat16 build has this kernel");
}

#endif
