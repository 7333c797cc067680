// Next-token choice on the device: greedy argmax and a finite check of the logits.
//
// The reference copies the whole logits row to the host and samples there
// (src/generation/generator.cpp:716-739, src/generation/sampler.cpp:43-148); here
// only the chosen ids cross.  Greedy: the largest logit, the lowest index among
// equals (src/generation/sampler.cpp:58-62).
#include "common.cuh"

namespace skv {

// One block per row.  flag |= 2 if a logit of the row is NaN or infinite
// (src/generation/sampler.cpp:52-56 rejects such rows).
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab,
                              int* __restrict__ flag) {
    __shared__ float best_value[32];
    __shared__ int best_index[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float value = -INFINITY;
    int index = 0x7fffffff;
    bool bad = false;
    auto consider = [&](float v, int c) {
        if (!isfinite(v)) bad = true;
        if (v > value || (v == value && c < index)) { value = v; index = c; }
    };
    if ((((uintptr_t)row) & 15) == 0) {
        const int quads = vocab >> 2;
        for (int i = threadIdx.x; i < quads; i += blockDim.x) {
            const float4 v = ((const float4*)row)[i];
            consider(v.x, 4 * i); consider(v.y, 4 * i + 1); consider(v.z, 4 * i + 2); consider(v.w, 4 * i + 3);
        }
        for (int c = (quads << 2) + threadIdx.x; c < vocab; c += blockDim.x) consider(row[c], c);
    } else {
        for (int c = threadIdx.x; c < vocab; c += blockDim.x) consider(row[c], c);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other_value > value || (other_value == value && other_index < index)) {
            value = other_value; index = other_index;
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && flag) atomicOr(flag, 2);
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        value = lane < warps ? best_value[lane] : -INFINITY;
        index = lane < warps ? best_index[lane] : 0x7fffffff;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
            if (other_value > value || (other_value == value && other_index < index)) {
                value = other_value; index = other_index;
            }
        }
        if (lane == 0) out[blockIdx.x] = index == 0x7fffffff ? 0 : index;
    }
}

}  // namespace skv

using namespace skv;

SKV_EXPORT int skv_argmax(const float* logits, int* out, int rows, int vocab, int* flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail("skv_argmax", "vocab must be positive");
    return launch_pdl("skv_argmax", argmax_kernel, dim3(rows), dim3(1024), 0, stream, logits, out, vocab, flag);
}

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling, one block per row.
//
// Same distribution as the reference's host sampler (src/generation/sampler.cpp:
// 64-147): logits / temperature; keep the k largest (equal values: lower index
// first); softmax; walking down that order keep tokens until the cumulative
// probability reaches top_p, the crossing token included; renormalise; draw.
// The order "larger value first, then lower index" is a 64-bit key; the k-th key
// and the key where the mass crosses top_p are found by radix selection (8 passes
// of 8 bits) instead of sorting.  Masses are summed as 40-bit fixed point in
// 64-bit integers, so sums do not depend on the order of additions: the same
// seed gives the same token whatever else is in the batch.  The draw is
// Philox4x32-10 keyed by the seed, with the counter (stream, position) the
// caller gives per row, and an inverse-CDF walk in index order.
namespace skv {

__device__ __forceinline__ uint32_t orderable(float v) {
    const uint32_t bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ unsigned long long sort_key(float v, int index) {
    return ((unsigned long long)orderable(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)index);
}

__device__ __forceinline__ unsigned long long fixed_mass(float v, float max_value) {
    // exp(v - max) in (0, 1] as 40-bit fixed point; never below 1 so that every kept token can be drawn
    const float w = expf(v - max_value);
    const unsigned long long q = (unsigned long long)(w * 1099511627776.0f);     // exact: a power of two
    return q ? q : 1ull;
}

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ uint32_t philox_first_word(unsigned long long seed, uint32_t stream, uint32_t position) {
    uint32_t c[4] = {position, stream, 0u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c[0];
}

constexpr int SAMPLE_THREADS = 512;

// Finds, among elements with key >= floor_key, the key where the running total of
// `what` (walking keys downward) first reaches `target`.  COUNT: what = 1 per
// element; otherwise what = fixed_mass.  Returns the key (every thread).
template <bool COUNT>
__device__ unsigned long long radix_select(const float* __restrict__ row, int vocab, float inv_scale_div,
                                           float max_value, unsigned long long floor_key,
                                           unsigned long long target, unsigned long long* hist,
                                           unsigned long long* shared_pick) {
    unsigned long long prefix = 0ull, remaining = target;
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
        __syncthreads();
        const unsigned long long high_mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i] / inv_scale_div;
            const unsigned long long key = sort_key(v, i);
            if (key < floor_key || (key & high_mask) != prefix) continue;
            const int bin = (int)((key >> shift) & 0xFFull);
            atomicAdd(&hist[bin], COUNT ? 1ull : fixed_mass(v, max_value));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long run = 0ull;
            int chosen = -1, lowest = 0;
            for (int b = 255; b >= 0; --b) {
                if (hist[b] == 0ull) continue;
                lowest = b;
                if (run + hist[b] >= remaining) { chosen = b; break; }
                run += hist[b];
            }
            if (chosen < 0) {
                // Cannot happen with integer masses (each level's bins add up to the bin
                // chosen above); if it did, keep everything down to the lowest key.
                chosen = lowest;
                shared_pick[1] = hist[lowest];
            } else {
                shared_pick[1] = remaining - run;
            }
            shared_pick[0] = (unsigned long long)chosen;
        }
        __syncthreads();
        prefix |= shared_pick[0] << shift;
        remaining = shared_pick[1];
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, float temperature, int top_k,
              float top_p, unsigned long long seed, const int* __restrict__ streams,
              const int* __restrict__ counters, int* __restrict__ flag) {
    __shared__ unsigned long long hist[256];
    __shared__ unsigned long long pick[2];
    __shared__ unsigned long long chunk_sum[SAMPLE_THREADS];
    __shared__ float scratch[33];
    __shared__ int bad_flag;
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    if (threadIdx.x == 0) bad_flag = 0;
    __syncthreads();

    // maximum of the scaled logits (and the finite check)
    float local_max = -INFINITY;
    bool bad = false;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i] / temperature;
        if (!isfinite(v)) bad = true;
        local_max = fmaxf(local_max, v);
    }
    if (bad) bad_flag = 1;
    local_max = warp_max(local_max);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = local_max;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : -INFINITY;
        m = warp_max(m);
        if (threadIdx.x == 0) scratch[32] = m;
    }
    __syncthreads();
    const float max_value = scratch[32];
    if (bad_flag) {
        if (threadIdx.x == 0) { if (flag) atomicOr(flag, 2); out[blockIdx.x] = 0; }
        return;
    }

    unsigned long long floor_key = 0ull;
    if (top_k > 0 && top_k < vocab)
        floor_key = radix_select<true>(row, vocab, temperature, max_value, 0ull, (unsigned long long)top_k, hist, pick);

    // total mass of what is allowed so far
    auto total_mass = [&](unsigned long long floor) {
        unsigned long long local = 0ull;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i] / temperature;
            if (sort_key(v, i) >= floor) local += fixed_mass(v, max_value);
        }
        __syncthreads();
        chunk_sum[threadIdx.x] = local;
        __syncthreads();
        for (int stride = SAMPLE_THREADS / 2; stride > 0; stride >>= 1) {
            if (threadIdx.x < stride) chunk_sum[threadIdx.x] += chunk_sum[threadIdx.x + stride];
            __syncthreads();
        }
        const unsigned long long total = chunk_sum[0];
        __syncthreads();
        return total;
    };

    if (top_p < 1.0f) {
        const unsigned long long total = total_mass(floor_key);
        unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        if (target < 1ull) target = 1ull;
        floor_key = radix_select<false>(row, vocab, temperature, max_value, floor_key, target, hist, pick);
    }

    // draw: inverse CDF over the survivors in index order, contiguous chunk per thread
    const int per_thread = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(vocab, (int)threadIdx.x * per_thread), end = min(vocab, begin + per_thread);
    unsigned long long mine = 0ull;
    for (int i = begin; i < end; ++i) {
        const float v = row[i] / temperature;
        if (sort_key(v, i) >= floor_key) mine += fixed_mass(v, max_value);
    }
    chunk_sum[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0ull;
        for (int t = 0; t < SAMPLE_THREADS; ++t) total += chunk_sum[t];
        const uint32_t r = philox_first_word(seed, (uint32_t)streams[blockIdx.x], (uint32_t)counters[blockIdx.x]);
        // target in [0, total): floor(total * r / 2^32) with a 96-bit product
        const unsigned long long hi = __umul64hi(total, (unsigned long long)r << 32);
        unsigned long long target = hi;
        unsigned long long run = 0ull;
        int owner = SAMPLE_THREADS - 1;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            if (target < run + chunk_sum[t]) { owner = t; break; }
            run += chunk_sum[t];
        }
        pick[0] = (unsigned long long)owner;
        pick[1] = target - run;
    }
    __syncthreads();
    if ((int)pick[0] == (int)threadIdx.x) {
        unsigned long long left = pick[1], run = 0ull;
        int chosen = -1, last_allowed = -1;
        for (int i = begin; i < end; ++i) {
            const float v = row[i] / temperature;
            if (sort_key(v, i) < floor_key) continue;
            last_allowed = i;
            run += fixed_mass(v, max_value);
            if (left < run) { chosen = i; break; }
        }
        out[blockIdx.x] = chosen >= 0 ? chosen : max(last_allowed, 0);
    }
}

}  // namespace skv

SKV_EXPORT int skv_sample(const float* logits, int* out, int rows, int vocab, float temperature, int top_k,
                          float top_p, unsigned long long seed, const int* streams, const int* counters,
                          int* flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail("skv_sample", "vocab must be positive");
    if (!(temperature > 0.0f) || !isfinite(temperature))
        return fail("skv_sample", "temperature must be positive and finite (0 is greedy: use skv_argmax)");
    if (top_k < 0) return fail("skv_sample", "top_k must be non-negative");
    if (!(top_p > 0.0f) || top_p > 1.0f) return fail("skv_sample", "top_p must be in (0, 1]");
    return launch_pdl("skv_sample", sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, out, vocab,
                      temperature, top_k, top_p, (unsigned long long)seed, streams, counters, flag);
}
