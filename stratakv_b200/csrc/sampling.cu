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
    // exp(v - max) in (0, 1] as 40-bit fixed point; never below 1 so that every kept token can be drawn.  (The
    // special-function unit's exponential, a few units in the last place of a float off libm's: a row is walked up to
    // twenty times and libm's expf was most of each walk.  Whatever it returns, every pass sees the same masses.)
    const float w = __expf(v - max_value);
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
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Finds, among elements with key >= floor_key, the key where the running total of
// `what` (walking keys downward) first reaches `target`.  COUNT: what = 1 per
// element; otherwise what = fixed_mass.  Returns the key (every thread).
// The histogram of a pass is filled a warp at a time: lanes whose elements fall in the same bin (most of a row does
// in the passes over the exponent bits) add up among themselves first and one of them adds to shared memory (every
// element for itself meant tens of thousands of atomic additions to three or four addresses a pass).  Masses are
// integers below 2^41, added as two halves of 20 bits so that the warp's 32-bit reduction serves.  When all 32 bits
// of the value are fixed and one element alone has that value there is no tie for the index bits to break: the last
// four passes are left out and the key's index bits stay zero, which keeps the same elements.
constexpr int SAMPLE_CANDIDATES = 4096;            // indices a block keeps once few enough elements are left in play

template <bool COUNT>
__device__ unsigned long long radix_select(const float* __restrict__ row, const float* scaled, int vocab, float inv_scale_div,
                                           float max_value, unsigned long long floor_key,
                                           unsigned long long target, unsigned long long* hist, unsigned int* members,
                                           unsigned long long* warp_hist, unsigned int* warp_members, int* candidates,
                                           unsigned long long* shared_pick, unsigned long long in_play) {
    // in_play: at most this many elements have a key >= floor_key (all of them: ~0)
    // warp_hist [warps][256], warp_members [warps][256]: a warp adds to its own histogram with plain reads and writes
    // (its leaders of one round hold different bins), and the histograms are added up after the walk: atomic additions
    // of sixteen warps to the two or three bins that a pass over the high bits fills cost more than the walk itself.
    // Only the elements of the bin that a pass chose are in play in the next one.  Once they are at most
    // SAMPLE_CANDIDATES, the next walk over the row writes their indices down (candidates; shared_pick[3] counts them),
    // and the passes after it walk that list instead of the row.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long* my_hist = warp_hist + warp * 256;
    unsigned int* my_members = warp_members + warp * 256;
    unsigned long long prefix = 0ull, remaining = target;
    int listed = -1;                                   // how many indices the list holds (-1: none yet)
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256 * SAMPLE_WARPS; b += blockDim.x) { warp_hist[b] = 0ull; warp_members[b] = 0u; }
        const bool collect = listed < 0 && in_play <= (unsigned long long)SAMPLE_CANDIDATES;
        if (threadIdx.x == 0) shared_pick[3] = 0ull;
        __syncthreads();
        const unsigned long long high_mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
        // one element a lane: `live` lanes bring an element (index i, scaled value v) that may or may not be in play
        auto account = [&](bool live, int i, float v) {
            bool valid = false;
            int bin = 0;
            unsigned long long mass = 0ull;
            if (live) {
                const unsigned long long key = sort_key(v, i);
                valid = key >= floor_key && (key & high_mask) == prefix;
                bin = (int)((key >> shift) & 0xFFull);
                if (!COUNT && valid) mass = fixed_mass(v, max_value);
            }
            const unsigned int voters = __ballot_sync(0xffffffffu, valid);
            if (voters == 0u) return;
            if (collect) {
                int slot = 0;
                if (lane == __ffs(voters) - 1) slot = (int)atomicAdd(&shared_pick[3], (unsigned long long)__popc(voters));
                slot = __shfl_sync(0xffffffffu, slot, __ffs(voters) - 1);
                if (valid) candidates[slot + __popc(voters & ((1u << lane) - 1u))] = i;
            }
            if (valid) {
                const unsigned int peers = __match_any_sync(voters, bin);
                const bool leader = (__ffs(peers) - 1) == lane;
                if (COUNT) {
                    if (leader) my_hist[bin] += (unsigned long long)__popc(peers);
                } else {
                    const unsigned int low = __reduce_add_sync(peers, (unsigned int)(mass & 0xFFFFFull));
                    const unsigned int high = __reduce_add_sync(peers, (unsigned int)(mass >> 20));
                    if (leader) {
                        my_hist[bin] += ((unsigned long long)high << 20) + low;
                        my_members[bin] += (unsigned int)__popc(peers);
                    }
                }
            }
            __syncwarp();                          // (a round's writes before the next round's reads of the same bins)
        };
        if (listed >= 0) {
            for (int base = (int)threadIdx.x - lane; base < listed; base += SAMPLE_THREADS) {
                const int c = base + lane;
                const bool live = c < listed;
                const int i = live ? candidates[c] : 0;
                const float v = live ? (scaled ? scaled[i] : row[i] / inv_scale_div) : 0.0f;
                account(live, i, v);
            }
        } else {
            for (int base4 = (int)threadIdx.x - lane; base4 < vocab; base4 += 4 * SAMPLE_THREADS) {   // the same trips for a warp's lanes
                float x[4];                                              // four loads on their way
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = base4 + u * SAMPLE_THREADS + lane;
                    x[u] = i < vocab ? (scaled ? scaled[i] : row[i]) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int base = base4 + u * SAMPLE_THREADS;
                    if (base >= vocab) break;
                    const int i = base + lane;
                    account(i < vocab, i, scaled ? x[u] : x[u] / inv_scale_div);
                }
            }
        }
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned long long total = 0ull;
            unsigned int count = 0u;
            for (int w = 0; w < SAMPLE_WARPS; ++w) { total += warp_hist[w * 256 + b]; count += warp_members[w * 256 + b]; }
            hist[b] = total;
            members[b] = count;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // Warp 0 finds the bin in which the running total, from bin 255 downwards, reaches `remaining`: lane l owns
            // bins 255 - 8l down to 248 - 8l (one thread walking all 256 bins took 4 us a pass).
            unsigned long long mine[8], own = 0ull;
#pragma unroll
            for (int j = 0; j < 8; ++j) { mine[j] = hist[255 - 8 * lane - j]; own += mine[j]; }
            unsigned long long upto = own;                               // lanes 0..lane, i.e. the higher bins and these
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned long long above = __shfl_up_sync(0xffffffffu, upto, offset);
                if (lane >= offset) upto += above;
            }
            const unsigned int reached = __ballot_sync(0xffffffffu, own > 0ull && upto >= remaining);
            const unsigned int holders = __ballot_sync(0xffffffffu, own > 0ull);
            if (reached) {
                if (lane == __ffs(reached) - 1) {
                    unsigned long long run = upto - own;                 // the total of the bins above this lane's
                    for (int j = 0; j < 8; ++j) {
                        if (mine[j] == 0ull) continue;
                        if (run + mine[j] >= remaining) {
                            const int chosen = 255 - 8 * lane - j;
                            shared_pick[0] = (unsigned long long)chosen;
                            shared_pick[1] = remaining - run;
                            shared_pick[2] = COUNT ? mine[j] : (unsigned long long)members[chosen];    // elements in that bin
                            break;
                        }
                        run += mine[j];
                    }
                }
            } else if (lane == (holders ? 31 - __clz(holders) : 0)) {
                // Cannot happen with integer masses (each level's bins add up to the bin
                // chosen above); if it did, keep everything down to the lowest key.
                int lowest = 255 - 8 * lane;
                for (int j = 0; j < 8; ++j) if (mine[j] != 0ull) lowest = 255 - 8 * lane - j;
                shared_pick[0] = (unsigned long long)lowest;
                shared_pick[1] = hist[lowest];
                shared_pick[2] = COUNT ? hist[lowest] : (unsigned long long)members[lowest];
            }
        }
        __syncthreads();
        prefix |= shared_pick[0] << shift;
        remaining = shared_pick[1];
        in_play = shared_pick[2];
        if (collect) listed = (int)shared_pick[3];
        __syncthreads();
        if (shift == 32 && in_play == 1ull) break;
    }
    return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, float temperature, int top_k,
              float top_p, unsigned long long seed, const int* __restrict__ streams,
              const int* __restrict__ counters, int* __restrict__ flag, int staged) {
    // `staged`: the row divided by the temperature is kept in (dynamic) shared memory after the first walk, and the
    // later walks read it there; rows too long for that are read and divided again each time, with the same results
    extern __shared__ __align__(16) unsigned char sample_smem[];
    unsigned long long* warp_hist = (unsigned long long*)sample_smem;             // [warps][256]
    unsigned int* warp_members = (unsigned int*)(warp_hist + SAMPLE_WARPS * 256);  // [warps][256]
    int* candidates = (int*)(warp_members + SAMPLE_WARPS * 256);                  // [SAMPLE_CANDIDATES]
    float* scaled = staged ? (float*)(candidates + SAMPLE_CANDIDATES) : nullptr;
    __shared__ unsigned long long hist[256];
    __shared__ unsigned int members[256];
    __shared__ unsigned long long pick[4];
    __shared__ unsigned long long warp_total[SAMPLE_WARPS];
    __shared__ float scratch[33];
    __shared__ int bad_flag;
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) bad_flag = 0;
    __syncthreads();

    // maximum of the scaled logits (and the finite check)
    float local_max = -INFINITY;
    bool bad = false;
    // (four loads on their way per thread: the row comes from L2 the first time)
    for (int i0 = threadIdx.x; i0 < vocab; i0 += 4 * SAMPLE_THREADS) {
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) x[u] = i0 + u * SAMPLE_THREADS < vocab ? row[i0 + u * SAMPLE_THREADS] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i0 + u * SAMPLE_THREADS < vocab) {
                const float v = x[u] / temperature;
                if (scaled) scaled[i0 + u * SAMPLE_THREADS] = v;
                if (!isfinite(v)) bad = true;
                local_max = fmaxf(local_max, v);
            }
        }
    }
    if (bad) bad_flag = 1;
    local_max = warp_max(local_max);
    if (lane == 0) scratch[warp] = local_max;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = threadIdx.x < SAMPLE_WARPS ? scratch[threadIdx.x] : -INFINITY;
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
        floor_key = radix_select<true>(row, scaled, vocab, temperature, max_value, 0ull, (unsigned long long)top_k, hist, members, warp_hist,
                                       warp_members, candidates, pick, ~0ull);

    // A warp owns a stretch of the row and each of its lanes a run of consecutive elements in it (a lane's loads walk
    // along cache lines that stay in L1).  A lane keeps the mass of what is allowed in its run; the warp's total goes
    // to warp_total.  Integer masses: the totals do not depend on who adds what.
    const int per_lane = ((vocab + SAMPLE_WARPS - 1) / SAMPLE_WARPS + 31) / 32;
    const int begin = min(vocab, (warp * 32 + lane) * per_lane), end = min(vocab, begin + per_lane);
    auto lane_mass = [&](unsigned long long floor) {
        unsigned long long local = 0ull;
        for (int i = begin; i < end; ++i) {
            const float v = scaled ? scaled[i] : row[i] / temperature;
            if (sort_key(v, i) >= floor) local += fixed_mass(v, max_value);
        }
        const unsigned long long total = warp_sum_u64(local);
        __syncthreads();                           // (whoever still reads the totals of a round before has done so)
        if (lane == 0) warp_total[warp] = total;
        __syncthreads();
        return local;
    };

    if (top_p < 1.0f) {
        lane_mass(floor_key);
        unsigned long long total = 0ull;
        for (int w = 0; w < SAMPLE_WARPS; ++w) total += warp_total[w];
        unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        if (target < 1ull) target = 1ull;
        floor_key = radix_select<false>(row, scaled, vocab, temperature, max_value, floor_key, target, hist, members, warp_hist,
                                        warp_members, candidates, pick, floor_key ? (unsigned long long)top_k : ~0ull);
    }

    // draw: the inverse of the cumulative masses of the survivors in index order: the warp, then the lane, then the
    // element in whose mass the drawn number falls
    const unsigned long long mine = lane_mass(floor_key);
    if (threadIdx.x == 0) {
        unsigned long long total = 0ull;
        for (int w = 0; w < SAMPLE_WARPS; ++w) total += warp_total[w];
        const uint32_t r = philox_first_word(seed, (uint32_t)streams[blockIdx.x], (uint32_t)counters[blockIdx.x]);
        // target in [0, total): floor(total * r / 2^32) with a 96-bit product
        const unsigned long long target = __umul64hi(total, (unsigned long long)r << 32);
        unsigned long long run = 0ull;
        int owner = SAMPLE_WARPS - 1;
        for (int w = 0; w < SAMPLE_WARPS; ++w) {
            if (target < run + warp_total[w]) { owner = w; break; }
            run += warp_total[w];
        }
        pick[0] = (unsigned long long)owner;
        pick[1] = target - run;
    }
    __syncthreads();
    if ((int)pick[0] == warp) {
        unsigned long long upto = mine;                                  // inclusive sum over lanes 0..lane
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const unsigned long long below = __shfl_up_sync(0xffffffffu, upto, offset);
            if (lane >= offset) upto += below;
        }
        const unsigned long long left = pick[1];
        const unsigned int crossed = __ballot_sync(0xffffffffu, mine > 0ull && left < upto);
        const unsigned int holders = __ballot_sync(0xffffffffu, mine > 0ull);
        // (no lane crossed: cannot happen with integer masses; the last lane that holds anything then gives its last element)
        const int owner_lane = crossed ? __ffs(crossed) - 1 : (holders ? 31 - __clz(holders) : 0);
        if (lane == owner_lane) {
            unsigned long long remaining = crossed ? left - (upto - mine) : ~0ull, run = 0ull;
            int chosen = -1, last_allowed = -1;
            for (int i = begin; i < end; ++i) {
                const float v = scaled ? scaled[i] : row[i] / temperature;
                if (sort_key(v, i) < floor_key) continue;
                last_allowed = i;
                run += fixed_mass(v, max_value);
                if (remaining < run) { chosen = i; break; }
            }
            out[blockIdx.x] = chosen >= 0 ? chosen : max(last_allowed, 0);
        }
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
    // a row of up to 38,912 logits is kept in shared memory between the kernel's walks over it
    const size_t row_bytes = (size_t)vocab * sizeof(float);
    const size_t histograms = (size_t)SAMPLE_WARPS * 256 * (sizeof(unsigned long long) + sizeof(unsigned int)) +
                              (size_t)SAMPLE_CANDIDATES * sizeof(int);      // 48 KB of histograms and 16 KB of indices
    const int staged = row_bytes <= 152 * 1024 ? 1 : 0;
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        (int)(histograms + 152 * 1024));
        if (status != cudaSuccess) return fail("skv_sample", cudaGetErrorString(status));
        configured = true;
    }
    return launch_pdl("skv_sample", sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), histograms + (staged ? row_bytes : 0), stream, logits, out,
                      vocab, temperature, top_k, top_p, (unsigned long long)seed, streams, counters, flag, staged);
}
