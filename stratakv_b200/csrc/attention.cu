// Causal grouped-query attention over the paged cache, one warp per (token, head).
//
// Replaces the reference's paged_attention_decode_kernel (src/cuda/gemm_cuda.cu:
// 304-429), which serves one query token, with a kernel for any number of new
// tokens per sequence: a token at absolute position p attends to cached keys
// lo..p of its own sequence (lo = 0, or p - window + 1 with a window), its own key
// included because the cache write runs first.  As in the reference,
// kv_head = q_head / (heads / kv_heads), the scale multiplies the finished dot
// product, and max, exp, sums and the weighted sum of values are in float
// (src/layers/attention.cpp:261-338); the softmax is the online form, by chunks of
// 32 keys.  expf is the accurate one: nothing here is built with fast-math.
//
// Cache layout per entry: [block][kv_head][block_size][head_dim]; a token's keys
// are found through block_table[seq][position / block_size].
#include "common.cuh"

namespace skv {

constexpr int HD = SKV_HEAD_DIM;
constexpr int DIMS_PER_LANE = (HD + 31) / 32;
constexpr int ATT_WARPS = 4;

template <typename T, int VEC> struct RowDot;

// dot(q, key row) with 16-byte loads of the row.
__device__ __forceinline__ float row_dot(const float* __restrict__ q, const float* __restrict__ row) {
    float sum = 0.0f;
#pragma unroll
    for (int d = 0; d < HD; d += 4) {
        const float4 k = *(const float4*)(row + d);
        sum = fmaf(q[d], k.x, sum);
        sum = fmaf(q[d + 1], k.y, sum);
        sum = fmaf(q[d + 2], k.z, sum);
        sum = fmaf(q[d + 3], k.w, sum);
    }
    return sum;
}

__device__ __forceinline__ float row_dot(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row) {
    float sum = 0.0f;
#pragma unroll
    for (int d = 0; d < HD; d += 8) {
        const uint4 raw = *(const uint4*)(row + d);
        const __nv_bfloat162* pairs = (const __nv_bfloat162*)&raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 k = __bfloat1622float2(pairs[i]);
            sum = fmaf(q[d + 2 * i], k.x, sum);
            sum = fmaf(q[d + 2 * i + 1], k.y, sum);
        }
    }
    return sum;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                 const int* __restrict__ token_seq, T* __restrict__ out, int n_tokens, int num_heads,
                 int num_kv_heads, int block_size, float scale, int window) {
    __shared__ __align__(16) float q_smem[ATT_WARPS][HD];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
    if (item >= (long long)n_tokens * num_heads) return;       // whole warps leave together
    const int t = (int)(item / num_heads), head = (int)(item % num_heads);
    const int kv_head = head / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_width;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    float* qs = q_smem[warp];
    const T* q_row = q + ((size_t)t * num_heads + head) * HD;
    for (int d = lane; d < HD; d += 32) qs[d] = to_float(q_row[d]);
    __syncwarp();

    float acc[DIMS_PER_LANE];
#pragma unroll
    for (int i = 0; i < DIMS_PER_LANE; ++i) acc[i] = 0.0f;
    float running_max = -INFINITY, running_sum = 0.0f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        int row = 0;                                   // row index in units of HD elements
        float score = -INFINITY;
        if (valid) {
            const int block = table[j / block_size];
            row = (block * num_kv_heads + kv_head) * block_size + (j % block_size);
            score = row_dot(qs, k_cache + (size_t)row * HD) * scale;
        }
        const float new_max = fmaxf(running_max, warp_max(score));
        const float p = valid ? expf(score - new_max) : 0.0f;
        const float rescale = expf(running_max - new_max);     // 0 on the first chunk
        running_sum = running_sum * rescale + warp_sum(p);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < DIMS_PER_LANE; ++i) acc[i] *= rescale;
        const int count = min(32, pos - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, row, jj);
            const T* v_row = v_cache + (size_t)rj * HD;
#pragma unroll
            for (int i = 0; i < DIMS_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < HD) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
            }
        }
    }
    T* out_row = out + ((size_t)t * num_heads + head) * HD;
    const float inverse = 1.0f / running_sum;
#pragma unroll
    for (int i = 0; i < DIMS_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < HD) out_row[d] = from_float<T>(acc[i] * inverse);
    }
}

}  // namespace skv

using namespace skv;

SKV_EXPORT int skv_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                             int table_width, const int* positions, const int* token_seq, void* out,
                             int n_tokens, int num_heads, int num_kv_heads, int head_dim, int block_size,
                             float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim != HD) return fail("skv_attention", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || window < 0) return fail("skv_attention", "bad block size or window");
    const long long items = (long long)n_tokens * num_heads;
    const long long blocks = (items + ATT_WARPS - 1) / ATT_WARPS;
    if (blocks > 0x7fffffffLL) return fail("skv_attention", "too many tokens in one step");
    return launch_pdl("skv_attention", attention_kernel<skv_t>, dim3((unsigned)blocks), dim3(ATT_WARPS * 32), 0,
                      stream, (const skv_t*)q, (const skv_t*)k_cache, (const skv_t*)v_cache, block_table,
                      table_width, positions, token_seq, (skv_t*)out, n_tokens, num_heads, num_kv_heads,
                      block_size, scale, window);
}
