// Decode attention for bfloat16: one new token per sequence, grouped-query heads
// sharing one pass over their KV head's cache, the context split across blocks.
//
// Replaces the reference's paged_attention_decode_kernel (src/cuda/gemm_cuda.cu:
// 304-429), which gives one block to each query head and walks the whole context
// serially with scalar dot products.  Here a block takes (sequence, KV head,
// context split); its G = heads / kv_heads query heads are the 16 rows of
// mma.sync m16n8k16 tiles (rows beyond G are zero), so every cached key and value
// is read once for all of them.  Scores, the online softmax and the output
// accumulate in float (src/layers/attention.cpp:261-338).  Each warp owns every
// W-th group of 16 keys; warps are merged in shared memory, splits by a second
// small kernel.  Split boundaries come from the sequence's own length.
//
// Fragment loading without shared memory: for Q.K^T a lane reads 4 consecutive
// head-dim elements of its key (8 bytes), which serve as the MMA's k indices
// {2t, 2t+1, 2t+8, 2t+9}; Q is loaded with the same permutation, so the dot
// products are unchanged.  For P.V a lane reads head_dim/8 consecutive elements of
// four keys and pairs them across keys with byte permutes; tile j's column g is
// then head-dim element g*head_dim/8 + j, undone when the output is written.
#include "common.cuh"

#include <mutex>

#if SKV_DTYPE == SKV_BF16

namespace skv {

constexpr int DHD = SKV_HEAD_DIM;
constexpr int KSTEPS = DHD / 16;          // k16 steps of Q.K^T
constexpr int OTILES = DHD / 8;           // n8 tiles of the output
constexpr int VWORDS = DHD / 16;          // 32-bit words a lane reads per key for P.V
constexpr int DEC_WARPS = 8;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2^x by the special-function unit; scores are kept in units of log2 (see attention_prefill.cu).
__device__ __forceinline__ float dec_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}

__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                        int table_width, const int* __restrict__ ctx_after, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ partial_o, float* __restrict__ partial_ml, int num_heads,
                        int num_kv_heads, int block_size, float scale, int window, int splits, int m_tiles) {
    extern __shared__ float merge[];                  // [warps][16][DHD + 2]
    constexpr int PITCH = DHD + 2;
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int seq = blockIdx.x;
    const int kv_head = blockIdx.y / m_tiles, m_tile = blockIdx.y - kv_head * m_tiles;
    const int split = blockIdx.z;
    const int group_size = num_heads / num_kv_heads;
    const int head0 = kv_head * group_size + m_tile * 16;
    const int rows = min(16, group_size - m_tile * 16);

    const int ctx = ctx_after[seq];                   // keys 0 .. ctx-1; the query sits at ctx-1
    const int lo = window > 0 ? max(0, ctx - window) : 0;
    const int first_group = lo >> 4, end_group = (ctx + 15) >> 4;
    const int per_split = (end_group - first_group + splits - 1) / splits;
    const int my_first = first_group + split * per_split;
    const int my_end = min(end_group, my_first + per_split);
    const int* table = block_table + (size_t)seq * table_width;
    const float scale_log2 = scale * 1.4426950408889634f;

    // Q fragments: rows g and g+8 are heads head0+g and head0+g+8; 4 head-dim elements per k16 step
    uint32_t qa[KSTEPS][4];
    {
        const __nv_bfloat16* q_seq = q + (size_t)seq * num_heads * DHD;
#pragma unroll
        for (int s = 0; s < KSTEPS; ++s) {
            uint2 top = make_uint2(0u, 0u), bottom = make_uint2(0u, 0u);
            if (g < rows) top = *(const uint2*)(q_seq + (size_t)(head0 + g) * DHD + 16 * s + 4 * tig);
            if (g + 8 < rows) bottom = *(const uint2*)(q_seq + (size_t)(head0 + g + 8) * DHD + 16 * s + 4 * tig);
            qa[s][0] = top.x; qa[s][1] = bottom.x; qa[s][2] = top.y; qa[s][3] = bottom.y;
        }
    }

    float o[OTILES][4];
#pragma unroll
    for (int j = 0; j < OTILES; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float row_max[2] = {-INFINITY, -INFINITY};        // rows g and g+8
    float row_sum[2] = {0.0f, 0.0f};                  // this lane's share; summed over the quad at the end

    for (int group = my_first + warp; group < my_end; group += DEC_WARPS) {
        const int j0 = group << 4;
        const int block = table[j0 / block_size];
        const size_t base = ((size_t)(block * num_kv_heads + kv_head) * block_size + (j0 % block_size)) * DHD;
        const __nv_bfloat16* k_rows = k_cache + base;
        const __nv_bfloat16* v_rows = v_cache + base;

        // values first (their loads do not depend on the scores): keys 2t, 2t+1, 2t+8, 2t+9
        uint32_t vw[4][VWORDS];
        {
            const int keys[4] = {2 * tig, 2 * tig + 1, 2 * tig + 8, 2 * tig + 9};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool live = j0 + keys[i] < ctx;
                const uint32_t* src = (const uint32_t*)(v_rows + (size_t)keys[i] * DHD + g * (DHD / 8));
#pragma unroll
                for (int w = 0; w < VWORDS; ++w) vw[i][w] = live ? src[w] : 0u;
            }
        }
        float s[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.0f;
            const bool live = j0 + 8 * t + g < ctx;
            const __nv_bfloat16* key_row = k_rows + (size_t)(8 * t + g) * DHD + 4 * tig;
#pragma unroll
            for (int step = 0; step < KSTEPS; ++step) {
                const uint2 kb = live ? *(const uint2*)(key_row + 16 * step) : make_uint2(0u, 0u);
                mma16816(s[t], qa[step][0], qa[step][1], qa[step][2], qa[step][3], kb.x, kb.y);
            }
        }
        // scale, mask, online softmax
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
            // a group can be fully masked for this row only through the window's lower edge
            corr[r] = new_max == -INFINITY ? 1.0f : dec_exp2(row_max[r] - new_max);
            row_max[r] = new_max;
        }
        float p[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float m = row_max[c >> 1];
                p[t][c] = m == -INFINITY ? 0.0f : dec_exp2(s[t][c] - m);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
            row_sum[r] = row_sum[r] * corr[r] + p[0][2 * r] + p[0][2 * r + 1] + p[1][2 * r] + p[1][2 * r + 1];
#pragma unroll
        for (int j = 0; j < OTILES; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        const uint32_t a0 = pack_bf16(p[0][0], p[0][1]), a1 = pack_bf16(p[0][2], p[0][3]);
        const uint32_t a2 = pack_bf16(p[1][0], p[1][1]), a3 = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
        for (int w = 0; w < VWORDS; ++w) {
            // low halves are element 2w of the lane's range, high halves element 2w+1
            mma16816(o[2 * w], a0, a1, a2, a3, __byte_perm(vw[0][w], vw[1][w], 0x5410),
                     __byte_perm(vw[2][w], vw[3][w], 0x5410));
            mma16816(o[2 * w + 1], a0, a1, a2, a3, __byte_perm(vw[0][w], vw[1][w], 0x7632),
                     __byte_perm(vw[2][w], vw[3][w], 0x7632));
        }
    }
    // merge the warps
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    float* mine = merge + (size_t)warp * 16 * PITCH;
#pragma unroll
    for (int j = 0; j < OTILES; ++j) {
        const int d0 = (2 * tig) * (DHD / 8) + j, d1 = (2 * tig + 1) * (DHD / 8) + j;
        mine[g * PITCH + d0] = o[j][0];
        mine[g * PITCH + d1] = o[j][1];
        mine[(g + 8) * PITCH + d0] = o[j][2];
        mine[(g + 8) * PITCH + d1] = o[j][3];
    }
    if (tig == 0) {
        mine[g * PITCH + DHD] = row_max[0];
        mine[g * PITCH + DHD + 1] = row_sum[0];
        mine[(g + 8) * PITCH + DHD] = row_max[1];
        mine[(g + 8) * PITCH + DHD + 1] = row_sum[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * DHD; idx += blockDim.x) {
        const int r = idx / DHD, d = idx - r * DHD;
        float m = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, merge[((size_t)w * 16 + r) * PITCH + DHD]);
        float total = 0.0f, sum = 0.0f;
        if (m != -INFINITY) {
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float* tile = merge + ((size_t)w * 16 + r) * PITCH;
                const float weight = dec_exp2(tile[DHD] - m);      // 0 for a warp that saw no key
                total += weight * tile[d];
                sum += weight * tile[DHD + 1];
            }
        }
        const int head = head0 + r;
        if (splits == 1) {
            out[((size_t)seq * num_heads + head) * DHD + d] = __float2bfloat16_rn(total / sum);
        } else {
            const size_t at = ((size_t)seq * num_heads + head) * splits + split;
            partial_o[at * DHD + d] = total;
            if (d == 0) { partial_ml[2 * at] = m; partial_ml[2 * at + 1] = sum; }
        }
    }
}

// out[seq, head, :] = sum_s e^(m_s - M) O_s / sum_s e^(m_s - M) l_s
__global__ void decode_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                      __nv_bfloat16* __restrict__ out, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t item = blockIdx.x;                   // seq * num_heads + head
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, partial_ml[2 * (item * splits + s)]);
    for (int d = threadIdx.x; d < DHD; d += blockDim.x) {
        float total = 0.0f, sum = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const size_t at = item * splits + s;
            const float ms = partial_ml[2 * at];
            if (ms == -INFINITY) continue;
            const float weight = dec_exp2(ms - m);
            total += weight * partial_o[at * DHD + d];
            sum += weight * partial_ml[2 * at + 1];
        }
        out[item * DHD + d] = __float2bfloat16_rn(total / sum);
    }
}

}  // namespace skv

using namespace skv;

// Scratch the caller provides when splits > 1: partial_o [n_seqs * heads * splits * head_dim] floats,
// partial_ml [n_seqs * heads * splits * 2] floats.
SKV_EXPORT int skv_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                    const int* block_table, int table_width, const int* ctx_after, void* out,
                                    float* partial_o, float* partial_ml, int n_seqs, int num_heads,
                                    int num_kv_heads, int head_dim, int block_size, float scale, int window,
                                    int splits, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (head_dim != DHD) return fail("skv_attention_decode", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_decode", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || block_size % 16 != 0)
        return fail("skv_attention_decode", "block_size must be a positive multiple of 16");
    if (splits < 1 || splits > 65535) return fail("skv_attention_decode", "bad number of splits");
    if (splits > 1 && (!partial_o || !partial_ml))
        return fail("skv_attention_decode", "splits need scratch memory");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
        return fail("skv_attention_decode", "operands must be 16-byte aligned");
    const int group_size = num_heads / num_kv_heads;
    const int m_tiles = (group_size + 15) / 16;
    const size_t smem = (size_t)DEC_WARPS * 16 * (DHD + 2) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(decode_attention_kernel,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_attention_decode", cudaGetErrorString(status));
        configured = true;
    }
    dim3 grid(n_seqs, num_kv_heads * m_tiles, splits);
    if (int code = launch_pdl("skv_attention_decode", decode_attention_kernel, grid, dim3(DEC_WARPS * 32), smem,
                              stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                              (const __nv_bfloat16*)v_cache, block_table, table_width, ctx_after,
                              (__nv_bfloat16*)out, partial_o, partial_ml, num_heads, num_kv_heads, block_size,
                              scale, window, splits, m_tiles))
        return code;
    if (splits > 1)
        return launch_pdl("skv_attention_decode(combine)", decode_combine_kernel, dim3(n_seqs * num_heads),
                          dim3(DHD >= 128 ? 128 : 64), 0, stream, (const float*)partial_o,
                          (const float*)partial_ml, (__nv_bfloat16*)out, splits);
    return 0;
}

// ---------------------------------------------------------------------------
// skv_attention_decode_no_alloc: the same split decode attention for callers that cannot
// allocate device memory (declared in stratakv_no_alloc.h; it has no counterpart in the
// reference).  The partial results of the context splits live in a fixed array that is part of
// this library's device image instead of in memory the caller hands in.
namespace skv {

// Floats of scratch held by every GPU that loads this library, until the process exits
// (4.5 MiB).  A call needs n_seqs * heads * splits * (head_dim + 2) of them.
constexpr size_t NO_ALLOC_SCRATCH_FLOATS = (size_t)9 << 17;
static __device__ __align__(256) float g_no_alloc_scratch[NO_ALLOC_SCRATCH_FLOATS];

constexpr int NO_ALLOC_MAX_DEVICES = 64;

}  // namespace skv

SKV_EXPORT long long skv_attention_decode_no_alloc_capacity() { return (long long)NO_ALLOC_SCRATCH_FLOATS; }

SKV_EXPORT int skv_attention_decode_no_alloc(const void* q, const void* k_cache, const void* v_cache,
                                             const int* block_table, int table_width, const int* ctx_after,
                                             void* out, int n_seqs, int num_heads, int num_kv_heads,
                                             int head_dim, int block_size, float scale, int window, int splits,
                                             cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (head_dim != DHD) return fail("skv_attention_decode_no_alloc", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_decode_no_alloc", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || block_size % 16 != 0)
        return fail("skv_attention_decode_no_alloc", "block_size must be a positive multiple of 16");
    if (splits < 1 || splits > 65535) return fail("skv_attention_decode_no_alloc", "bad number of splits");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
        return fail("skv_attention_decode_no_alloc", "operands must be 16-byte aligned");
    const size_t slots = (size_t)n_seqs * num_heads * splits;
    const size_t needed = slots * (DHD + 2);
    if (needed > NO_ALLOC_SCRATCH_FLOATS) {
        char detail[256];
        snprintf(detail, sizeof detail,
                 "n_seqs * heads * splits * (head_dim + 2) = %zu floats of scratch are needed, the built-in "
                 "array holds %zu: use fewer splits or sequences per call",
                 needed, (size_t)NO_ALLOC_SCRATCH_FLOATS);
        return fail("skv_attention_decode_no_alloc", detail);
    }
    // In host code the array's name is a stand-in, not a device address.  The address the kernel
    // needs is asked for once per device, with that device current (the first call on a device
    // does it, which is why that call should come before any stream capture).
    // The per-device records below are read and written under one host lock, so that two host threads
    // making their first call at once do not race on them.
    static std::mutex setup_lock;
    static float* scratch_of_device[NO_ALLOC_MAX_DEVICES] = {nullptr};
    static bool attribute_set[NO_ALLOC_MAX_DEVICES] = {false};
    std::lock_guard<std::mutex> setup_guard(setup_lock);
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return fail("skv_attention_decode_no_alloc", cudaGetErrorString(status));
    if (device < 0 || device >= NO_ALLOC_MAX_DEVICES)
        return fail("skv_attention_decode_no_alloc", "device index is beyond what this entry point tracks");
    if (!scratch_of_device[device]) {
        float* address = nullptr;
        status = cudaGetSymbolAddress((void**)&address, g_no_alloc_scratch);
        if (status != cudaSuccess) return fail("skv_attention_decode_no_alloc(cudaGetSymbolAddress)", cudaGetErrorString(status));
        if (!address) return fail("skv_attention_decode_no_alloc", "cudaGetSymbolAddress returned no address");
        scratch_of_device[device] = address;
    }
    float* partial_o = scratch_of_device[device];
    float* partial_ml = partial_o + slots * DHD;
    const int group_size = num_heads / num_kv_heads;
    const int m_tiles = (group_size + 15) / 16;
    const size_t smem = (size_t)DEC_WARPS * 16 * (DHD + 2) * sizeof(float);
    if (!attribute_set[device]) {
        status = cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_attention_decode_no_alloc", cudaGetErrorString(status));
        attribute_set[device] = true;
    }
    // Every slot that the combine step reads is written by exactly one block of the first kernel
    // (a split without keys writes an empty partial), so nothing of the array has to start at zero.
    dim3 grid(n_seqs, num_kv_heads * m_tiles, splits);
    if (int code = launch_pdl("skv_attention_decode_no_alloc", decode_attention_kernel, grid, dim3(DEC_WARPS * 32),
                              smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                              (const __nv_bfloat16*)v_cache, block_table, table_width, ctx_after,
                              (__nv_bfloat16*)out, partial_o, partial_ml, num_heads, num_kv_heads, block_size,
                              scale, window, splits, m_tiles))
        return code;
    if (splits > 1)
        return launch_pdl("skv_attention_decode_no_alloc(combine)", decode_combine_kernel,
                          dim3(n_seqs * num_heads), dim3(DHD >= 128 ? 128 : 64), 0, stream,
                          (const float*)partial_o, (const float*)partial_ml, (__nv_bfloat16*)out, splits);
    return 0;
}

#else

SKV_EXPORT int skv_attention_decode(const void*, const void*, const void*, const int*, int, const int*, void*,
                                    float*, float*, int, int, int, int, int, float, int, int, cudaStream_t) {
    return skv::fail("skv_attention_decode", "the float32 build decodes with skv_attention");
}

SKV_EXPORT long long skv_attention_decode_no_alloc_capacity() { return 0; }

SKV_EXPORT int skv_attention_decode_no_alloc(const void*, const void*, const void*, const int*, int, const int*, void*,
                                             int, int, int, int, int, float, int, int, cudaStream_t) {
    return skv::fail("skv_attention_decode_no_alloc", "only the bfloat16 build has this kernel");
}

#endif
